"""Request-level sampling parameters and the host sampler chain over device top-k candidates.

The reference runs its sampler chain on the host (src/llama-sampling.cpp) over either the full
logits or, with ``presample_count = k``, over the k candidates a device top-k returned
(src/llama-execute-decode.cpp:132-154; common/sampling_local.cpp:109-125).  Here greedy requests are
sampled entirely on the device (argmax kernel inside the CUDA graph); everything else goes through
the device top-k and then this chain, whose order and defaults follow common/sampling_local.cpp:
153-209 and common/common_local.h:94-140: penalties -> top_k -> typical -> top_p -> min_p -> xtc ->
temperature -> logit_bias -> dist.  The native chain in ``libjib200_runtime.so`` implements the same
stages for the C API; this module is the engine-side implementation.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


@dataclass
class SamplingParams:
    temperature: float = 0.0          # <= 0: greedy (src/llama-sampling.cpp:246-263)
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    typical_p: float = 1.0
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    repeat_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 64
    logit_bias: Dict[int, float] = field(default_factory=dict)
    dynatemp_range: float = 0.0       # > 0: temperature +- range scaled by the normalised entropy ** dynatemp_exponent
    dynatemp_exponent: float = 1.0
    dry_multiplier: float = 0.0       # > 0 enables the "don't repeat yourself" penalty
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_penalty_last_n: int = -1
    min_keep: int = 0
    grammar: Optional[str] = None     # GBNF text: candidates that cannot continue it are dropped (needs the native chain)
    logprobs: bool = False            # report the log-probability of every generated token ...
    top_logprobs: int = 0             # ... and of this many most likely alternatives (at most the device top-k width)
    seed: Optional[int] = None
    max_tokens: int = -1
    ignore_eos: bool = False
    n_keep: Optional[int] = None      # head tokens kept if the prompt must be cut to fit (None: engine default; <0: all that fits)
    stop: List[str] = field(default_factory=list)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 and self.repeat_penalty == 1.0 and self.frequency_penalty == 0.0 \
            and self.presence_penalty == 0.0 and not self.logit_bias and not self.grammar


class HostSampler:
    """Per-request sampler state (RNG + token history for the penalties)."""

    def __init__(self, params: SamplingParams):
        self.p = params
        self.rng = np.random.Generator(np.random.PCG64(params.seed if params.seed is not None else None))
        self.history: List[int] = []

    def accept(self, token: int):
        self.history.append(int(token))
        if self.p.repeat_last_n > 0 and len(self.history) > self.p.repeat_last_n:
            del self.history[: len(self.history) - self.p.repeat_last_n]

    def sample(self, values: np.ndarray, ids: np.ndarray) -> int:
        """values/ids: candidate logits (any order) and their token ids."""
        p = self.p
        logit = values.astype(np.float64).copy()
        ids = ids.astype(np.int64)
        # penalties (src/llama-sampling.cpp:1284-1316)
        if self.history and (p.repeat_penalty != 1.0 or p.frequency_penalty or p.presence_penalty):
            counts: Dict[int, int] = {}
            for t in self.history:
                counts[t] = counts.get(t, 0) + 1
            for i, t in enumerate(ids):
                c = counts.get(int(t))
                if c:
                    logit[i] = logit[i] / p.repeat_penalty if logit[i] > 0 else logit[i] * p.repeat_penalty
                    logit[i] -= c * p.frequency_penalty + p.presence_penalty
        for t, b in p.logit_bias.items():
            hit = np.nonzero(ids == t)[0]
            if hit.size:
                logit[hit] += b
        if p.temperature <= 0.0:
            return int(ids[int(np.argmax(logit))])
        order = np.argsort(-logit, kind="stable")
        logit, ids = logit[order], ids[order]
        if p.top_k > 0:
            logit, ids = logit[: p.top_k], ids[: p.top_k]

        def softmax(x):
            e = np.exp(x - x.max())
            return e / e.sum()

        if p.typical_p < 1.0:
            pr = softmax(logit)
            ent = -(pr * np.log(pr + 1e-30)).sum()
            dev = np.abs(-np.log(pr + 1e-30) - ent)
            o = np.argsort(dev, kind="stable")
            keep = int(np.searchsorted(np.cumsum(pr[o]), p.typical_p) + 1)
            sel = np.sort(o[: max(1, keep)])
            logit, ids = logit[sel], ids[sel]
        if p.top_p < 1.0:
            pr = softmax(logit)
            keep = int(np.searchsorted(np.cumsum(pr), p.top_p) + 1)     # smallest prefix with cum >= top_p
            logit, ids = logit[: max(1, keep)], ids[: max(1, keep)]
        if p.min_p > 0.0:
            keep = logit >= logit.max() + math.log(p.min_p)
            logit, ids = logit[keep], ids[keep]
        if p.xtc_probability > 0.0 and self.rng.random() < p.xtc_probability:
            pr = softmax(logit)
            above = np.nonzero(pr >= p.xtc_threshold)[0]
            if above.size >= 2:
                logit, ids = logit[above[-1]:], ids[above[-1]:]
        pr = softmax(logit / p.temperature)
        return int(ids[int(self.rng.choice(len(ids), p=pr))])


class NativeSampler:
    """The same per-request sampler over the C++ chain of ``libllama.so`` (``csrc/capi/samplers.cpp``), built in the
    reference's order: penalties, dry, top_k, typical_p, top_p, min_p, xtc, temperature (entropy-scaled when
    ``dynatemp_range`` > 0), then logit_bias and dist (common/sampling_local.cpp:128-210).  Candidates are the device's
    top-k, as with the reference's presample path."""

    def __init__(self, params: SamplingParams, n_vocab: int = 0, n_ctx_train: int = 4096, token_table=None):
        """``token_table``: (pieces: list of bytes per token id, eog ids, eos id) -- needed only for ``params.grammar``."""
        import ctypes as C
        from .. import capi
        self.C, self.capi = C, capi
        L = self.L = capi.load()
        p = self.p = params
        seed = p.seed if p.seed is not None else 0xFFFFFFFF
        ch = self.chain = L.llama_sampler_chain_init(capi.SamplerChainParams(True))
        add = lambda smpl: L.llama_sampler_chain_add(ch, smpl)
        if p.grammar:
            if token_table is None:
                raise ValueError("a grammar needs the token texts (token_table)")
            pieces, eog, eos = token_table
            arr = (C.c_char_p * len(pieces))(*pieces)
            lens = (C.c_int32 * len(pieces))(*[len(b) for b in pieces])
            eog_a = (capi.llama_token * max(1, len(eog)))(*eog)
            g = L.jib_sampler_init_grammar_pieces(arr, lens, len(pieces), eog_a, len(eog), int(eos), p.grammar.encode(), b"root")
            if not g:
                raise ValueError("the grammar does not parse")
            add(g)                    # first: the other samplers then work on admissible candidates only
        add(L.llama_sampler_init_penalties(p.repeat_last_n, p.repeat_penalty, p.frequency_penalty, p.presence_penalty))
        if p.dry_multiplier > 0:
            add(L.llama_sampler_init_dry(None, n_ctx_train, p.dry_multiplier, p.dry_base, p.dry_allowed_length, p.dry_penalty_last_n,
                                         None, 0))
        if p.temperature > 0:
            add(L.llama_sampler_init_top_k(p.top_k))
            add(L.llama_sampler_init_typical(p.typical_p, p.min_keep))
            add(L.llama_sampler_init_top_p(p.top_p, p.min_keep))
            add(L.llama_sampler_init_min_p(p.min_p, p.min_keep))
            add(L.llama_sampler_init_xtc(p.xtc_probability, p.xtc_threshold, p.min_keep, seed & 0xFFFFFFFF))
            add(L.llama_sampler_init_temp_ext(p.temperature, p.dynatemp_range, p.dynatemp_exponent))
        if p.logit_bias:
            arr = (capi.LogitBias * len(p.logit_bias))(*[(int(t), float(b)) for t, b in p.logit_bias.items()])
            add(L.llama_sampler_init_logit_bias(n_vocab, len(p.logit_bias), arr))
        add(L.llama_sampler_init_dist(seed & 0xFFFFFFFF) if p.temperature > 0 else L.llama_sampler_init_greedy())
        self._buf = None

    def __del__(self):
        try:
            if self.chain:
                self.L.llama_sampler_free(self.chain)
                self.chain = None
        except Exception:
            pass

    def accept(self, token: int):
        self.L.llama_sampler_accept(self.chain, int(token))

    def sample(self, values: np.ndarray, ids: np.ndarray) -> int:
        n = len(ids)
        if self._buf is None or len(self._buf) < n:
            self._buf = (self.capi.TokenData * n)()
        buf = self._buf
        for i in range(n):
            buf[i].id, buf[i].logit, buf[i].p = int(ids[i]), float(values[i]), 0.0
        arr = self.capi.TokenDataArray(self.C.cast(buf, self.C.POINTER(self.capi.TokenData)), n, -1, False)
        self.L.llama_sampler_apply(self.chain, self.C.byref(arr))
        return int(arr.data[arr.selected].id)


def device_samplable(p: SamplingParams) -> bool:
    """True when a request needs only what the on-device sampler implements: top-k, top-p, min-p, temperature and a seeded
    draw (``ops.sample_topk``).  Penalties, DRY, grammar, logit bias, typical and XTC sampling need the host chain."""
    return (p.temperature > 0.0 and p.repeat_penalty == 1.0 and p.frequency_penalty == 0.0 and p.presence_penalty == 0.0
            and not p.logit_bias and p.typical_p >= 1.0 and p.xtc_probability <= 0.0 and p.dynatemp_range <= 0.0
            and p.dry_multiplier <= 0.0 and not p.grammar and p.min_keep <= 1)


class DeviceSampler:
    """Host half of the on-device sampler: the request's truncation settings and its random stream.  Every step in which
    the request has an output row takes one uniform number from the stream; it travels to the device with the step's
    other inputs, so the draw depends on the seed and the step count only -- not on when the host reads the result."""

    def __init__(self, params: SamplingParams):
        self.p = params
        self.rng = np.random.Generator(np.random.PCG64(params.seed if params.seed is not None else None))      # None: OS entropy

    def row(self) -> tuple:
        p = self.p
        return (float(p.temperature), float(p.top_k), float(p.top_p), float(p.min_p), float(self.rng.random()))

    def accept(self, token: int) -> None:
        pass

    def sample_host(self, values: np.ndarray, ids: np.ndarray, row: tuple) -> int:
        """The same draw on the host (a step whose other requests need the host chain hands out candidates, not ids)."""
        import torch

        from ..ops import reference as ref
        v = torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32))[None]
        i = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int32))[None]
        return int(ref.sample_topk(v, i, torch.tensor([row], dtype=torch.float32))[0])


def make_sampler(params: SamplingParams, n_vocab: int = 0, n_ctx_train: int = 4096, token_table=None):
    """The native chain unless it cannot be loaded or ``JITTORINFER_SAMPLER=python`` asks for the numpy one."""
    import os
    if params.grammar:
        return NativeSampler(params, n_vocab, n_ctx_train, token_table)      # no fallback: the numpy chain has no grammar
    if os.environ.get("JITTORINFER_SAMPLER", "native").lower() != "python":
        try:
            return NativeSampler(params, n_vocab, n_ctx_train)
        except Exception:      # library not built / not loadable: the numpy chain has the same semantics minus dry and dynatemp
            pass
    return HostSampler(params)
