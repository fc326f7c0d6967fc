"""The serving engine: scheduler -> packed step inputs -> model forward (CUDA graph or eager) -> sample.

One ``LLMEngine.step()`` is what one ``llama_decode`` + sampling round is in the reference
(src/llama-execute-decode.cpp:156-344 driven by examples/server/server.cpp:1304-1564).  Differences
by design:

* the batch description (tokens, positions, slot mapping, block tables, sequence lengths) is written
  by the native scheduler straight into ONE pinned host buffer and reaches the device with ONE
  async copy per step — no host-built masks (src/llama-context.cpp:244-518);
* decode-only batches replay a CUDA graph captured per batch bucket (the analogue of the reference's
  persistent GE graph, src/llama-context-load-utils.cpp:134-174), with padding rows masked by
  ``slot_mapping = -1`` / ``seq_len = 0``;
* greedy sampling stays on the device (argmax kernel in the graph); other requests use a device
  top-k ("presample", src/llama-execute-decode.cpp:132-154) followed by the host chain.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..utils import fault
from ..utils.trace import PhaseTimer, Tracer
from ..models.deepseek2 import DeepSeek2Model, ForwardBatch
from ..models.hparams import DeepSeek2HParams
from .native_rt import PagedKV, Scheduler, StepArrays, i32p
from .sampling import DeviceSampler, SamplingParams, device_samplable, make_sampler


@dataclass
class EngineConfig:
    n_ctx: int = 16384                 # total cached tokens over all sequences (reference: n_ctx cell pool)
    n_batch: int = 2048                # token budget of one step (chunked prefill)
    n_parallel: int = 8                # concurrent sequences (slots)
    n_ctx_slot: Optional[int] = None   # per-sequence limit; default n_ctx / n_parallel as in the reference
    block_size: int = 64
    n_keep: int = 0
    cont_batching: bool = True
    presample_count: int = 64
    cuda_graphs: bool = True
    graph_buckets: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64)
    defrag_thold: float = -1.0         # <0 disables automatic defrag
    mixed_prompt_budget: int = 0       # most prompt tokens per step while sequences are generating (0 = n_batch): bounds
                                       # the token-to-token latency of running requests during somebody else's prefill
    device_sampling: bool = False      # requests that need only top-k / top-p / min-p / temperature are sampled on the device
                                       # (ops.sample_topk; also JITTORINFER_DEVICE_SAMPLING=1); the others use the host chain
    run_ahead: bool = False            # greedy requests: launch decode step k+1 before the ids of step k reach the host
                                       # (also JITTORINFER_RUN_AHEAD=1)
    defrag_max_moves: int = 256


@dataclass
class RequestState:
    req_id: int
    params: SamplingParams
    sampler: Optional[object]          # NativeSampler or HostSampler
    n_prompt: int
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    dev: Optional[DeviceSampler] = None    # sampled on the device (then sampler is None)
    n_cached: int = 0                      # prompt tokens that were found in the cache (own slot or another sequence's blocks)
    logprobs: List[Tuple[int, float, List[Tuple[int, float]]]] = field(default_factory=list)
    # per generated token (params.logprobs): (token id, its log-probability, [(id, log-probability)] of the top alternatives)


@dataclass
class _InFlight:
    """A launched step whose sampled ids have not been read yet."""
    out: torch.Tensor                  # device ids (a graph's static output or an eager result)
    host: torch.Tensor                 # pinned buffer the ids are being copied into
    event: Optional[object]            # CUDA event after that copy (None on the CPU)
    n_out: int
    out_slots: np.ndarray              # scheduler slot of each output row
    status: Optional[torch.Tensor] = None   # pinned copy of the device status words taken behind this step


class _StepIO:
    """Packed int32 step inputs: a pinned host buffer, its device twin and typed views of both."""

    def __init__(self, cap_tokens: int, cap_seqs: int, max_blocks: int, device: torch.device):
        self.cap_tokens, self.cap_seqs, self.max_blocks = cap_tokens, cap_seqs, max_blocks
        sizes = [("tokens", cap_tokens), ("positions", cap_tokens), ("slot_mapping", cap_tokens),
                 ("q_start", cap_seqs + 1), ("seq_lens", cap_seqs), ("out_rows", cap_seqs),
                 ("block_tables", cap_seqs * max_blocks), ("samp", cap_seqs * 5),      # samp: fp32 sampling rows, bit-cast
                 ("seq_slots", cap_seqs), ("out_slots", cap_seqs)]
        off = 0
        self.off: Dict[str, Tuple[int, int]] = {}
        for name, n in sizes:
            self.off[name] = (off, n)
            off = (off + n + 3) // 4 * 4           # keep every section 16-byte aligned
        self.total = off
        # seq_slots / out_slots are host-only: the device copy stops before them
        self.dev_len = self.off["seq_slots"][0]
        pin = device.type == "cuda"
        self._pin = pin
        self.dev = torch.zeros(self.dev_len, dtype=torch.int32, device=device)
        self.d = {k: self.dev[o:o + n] for k, (o, n) in self.off.items() if o < self.dev_len}
        self._stages = [self._make_stage()]
        self.use_stage(0)

    def _make_stage(self):
        host = torch.zeros(self.total, dtype=torch.int32, pin_memory=self._pin)
        arr = host.numpy()
        h = {k: arr[o:o + n] for k, (o, n) in self.off.items()}
        arrays = StepArrays()
        for k in ("tokens", "positions", "slot_mapping", "q_start", "seq_lens", "seq_slots", "block_tables", "out_rows",
                  "out_slots"):
            setattr(arrays, k, h[k].ctypes.data_as(i32p))
        arrays.cap_tokens, arrays.cap_seqs, arrays.max_blocks_per_seq = self.cap_tokens, self.cap_seqs, self.max_blocks
        return host, arr, h, arrays

    def use_stage(self, i: int) -> None:
        """Selects the pinned host buffer the next step is assembled in.  A second stage exists only when the engine runs
        one step ahead: the asynchronous upload of step k may still be reading its buffer while step k + 1 is assembled."""
        while len(self._stages) <= i:
            self._stages.append(self._make_stage())
        self.host, self.np, self.h, self.arrays = self._stages[i]

    def upload(self):
        self.dev.copy_(self.host[: self.dev_len], non_blocking=True)

    @property
    def h2d_bytes(self) -> int:
        return self.dev_len * 4


class SplitCache:
    """Latent cache of a layer-split model: one [layers-on-device, n_slots, row] tensor per device; ``cache[il]`` is the
    layer's slice on its own device."""

    def __init__(self, layer_dev, n_slots: int, row: int, dtype, block_size: int):
        self.block_size = block_size
        self.by_dev: Dict[torch.device, torch.Tensor] = {}
        self.index: List[Tuple[torch.device, int]] = []
        counts: Dict[torch.device, int] = {}
        for d in layer_dev:
            self.index.append((d, counts.get(d, 0)))
            counts[d] = counts.get(d, 0) + 1
        for d, n in counts.items():
            self.by_dev[d] = torch.zeros(n, n_slots, row, dtype=dtype, device=d)

    def __getitem__(self, il: int) -> torch.Tensor:
        d, i = self.index[il]
        return self.by_dev[d][i]

    def copy_blocks(self, src: np.ndarray, dst: np.ndarray) -> None:
        for d, t in self.by_dev.items():
            s = torch.from_numpy(np.ascontiguousarray(src)).to(d)
            e = torch.from_numpy(np.ascontiguousarray(dst)).to(d)
            if d.type == "cuda":
                with torch.cuda.device(d):
                    ops.kv_block_copy(t, s, e, self.block_size)
            else:
                ops.kv_block_copy(t, s, e, self.block_size)


class LLMEngine:
    def __init__(self, model: DeepSeek2Model, cfg: EngineConfig = EngineConfig()):
        self.model = model
        self.cfg = cfg
        self.hp: DeepSeek2HParams = model.hp
        self.device = model.device
        bs = cfg.block_size
        self.n_ctx_slot = cfg.n_ctx_slot or max(bs, cfg.n_ctx // cfg.n_parallel)
        self.max_blocks = (self.n_ctx_slot + bs - 1) // bs
        self.n_blocks = max((cfg.n_ctx + bs - 1) // bs, self.max_blocks)
        if self.n_ctx_slot > model.max_positions:
            raise ValueError(f"n_ctx_slot {self.n_ctx_slot} exceeds the model's RoPE table ({model.max_positions})")
        self.kv = PagedKV(self.n_blocks, bs, cfg.n_parallel)
        self.sched = Scheduler(self.kv, cfg.n_parallel, cfg.n_batch, self.n_ctx_slot, self.hp.eos_id, cfg.n_keep,
                               cfg.cont_batching)
        if cfg.mixed_prompt_budget > 0:
            self.sched.set_mixed_prompt_budget(cfg.mixed_prompt_budget)
        if getattr(model, "split", False):
            self.kv_cache = SplitCache(model.layer_dev, self.n_blocks * bs, self.hp.kv_row, model.dtype, bs)
        else:
            self.kv_cache = torch.zeros(self.hp.n_layer, self.n_blocks * bs, self.hp.kv_row, dtype=model.dtype,
                                        device=self.device)
        cap_tokens = max(cfg.n_batch, max(cfg.graph_buckets))
        cap_seqs = max(cfg.n_parallel, max(cfg.graph_buckets))
        self.io = _StepIO(cap_tokens, cap_seqs, self.max_blocks, self.device)
        self.requests: Dict[int, RequestState] = {}
        self._next_id = 1
        self._graphs: Dict[Tuple[int, str], Tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self._use_graphs = cfg.cuda_graphs and self.device.type == "cuda" and not getattr(model, "split", False)
        self._out_host = torch.zeros(cap_seqs * (1 + 2 * max(1, cfg.presample_count)), dtype=torch.int32,
                                     pin_memory=self.device.type == "cuda")
        self.stats = {"steps": 0, "graph_steps": 0, "eager_steps": 0, "tokens_in": 0, "tokens_out": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "defrag_moves": 0}
        self.graph_launches: Dict[Tuple[int, str], int] = {}    # launcher calls captured per decode graph
        self.launches = 0                                          # launcher calls executed (eager + replayed)
        # Data-parallel attention + expert parallelism: every rank schedules its own requests, but the MoE layers are
        # collective, so all ranks step together; a rank without tokens runs the idle forward.  Each step all-reduces
        # an "I still have work" flag (the reference gathers per-rank token counts every decode for the same purpose,
        # src/llama-context.cpp:538-556).
        spec = getattr(model, "spec", None)
        self.dp = bool(spec is not None and spec.dp_attention and spec.sharded)
        self.dp_active = spec.tp_size if self.dp else 0
        self._dp_flag = torch.zeros(1, dtype=torch.int32, device=self.device) if self.dp else None
        self._idle_graph = None
        self.tracer = Tracer()            # JSON-lines step trace when JITTORINFER_TRACE names a file
        self._pressure = False            # free KV blocks held back by the kv_alloc fault site
        self._device_sampling = bool(cfg.device_sampling or os.environ.get("JITTORINFER_DEVICE_SAMPLING", "") == "1")
        self._run_ahead = bool(cfg.run_ahead or os.environ.get("JITTORINFER_RUN_AHEAD", "") == "1") and not self.dp \
            and not getattr(model, "split", False)
        self._inflight: Optional[_InFlight] = None
        self._stage = 0
        # Kernels that give up on a bounded wait (an mbarrier, a peer's flag) or catch an index out of range record it in
        # four status words on the device and carry on.  The engine copies them to pinned memory behind every step's ids
        # (same stream, no extra synchronisation) and fails the step when a code is set: nothing computed from such a step
        # is sampled or sent to a client; the caller resets the engine (the server answers 503 and keeps serving).
        self._status_dev = None
        self._status_hosts = None
        if self.device.type == "cuda" and not ops.force_torch() and not getattr(model, "split", False):
            self._status_dev = ops.nat().workspace(self.device).status
            self._status_hosts = [torch.zeros(4, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._out_hosts = [self._out_host, torch.zeros_like(self._out_host).pin_memory() if self.device.type == "cuda"
                           else torch.zeros_like(self._out_host)] if self._run_ahead else [self._out_host]
        self._flip = 0
        # Debug aid: JITTORINFER_KV_POISON=1 fills every cache block with NaN when its last reference goes away and checks the
        # logits of every (then eager) step: a read through a stale block table cannot pass unnoticed.
        self._poison = os.environ.get("JITTORINFER_KV_POISON", "") == "1"
        if self._poison:
            self.kv.track_freed(True)
            self._use_graphs = False
            self.stats["poisoned_blocks"] = 0
        from ..utils import graphdump
        il = graphdump.requested_layer()  # LLAMA_PRINT_LAYER=<il>: the first step writes that layer's op graph as dot text
        if il is not None:
            graphdump.dump_on_first_step(self, il)
        # Loading the weights takes seconds and not the same time on every rank; the in-kernel collectives give a peer about
        # a second before they report a silent peer.  Start the first step together.
        if getattr(model, "comm", None) is not None or getattr(self, "dp", False):
            self._host_barrier()

    # ------------------------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        if len(prompt) and (min(prompt) < 0 or max(prompt) >= self.hp.n_vocab):
            raise ValueError(f"prompt token ids must be in [0, {self.hp.n_vocab})")
        rid = self._next_id
        self._next_id += 1
        spec = getattr(self.model, "spec", None)
        if params.seed is None and not params.greedy and spec is not None and spec.sharded and not spec.dp_attention:
            # tensor/expert-parallel ranks each run the sampler over identical logits: an unseeded request gets a seed
            # that every rank derives alike (request ids advance in lockstep), or the ranks would draw different tokens
            params = SamplingParams(**{**params.__dict__, "seed": (0x9E3779B97F4A7C15 * rid + 0x1234567) & 0xFFFFFFFF})
        dev = DeviceSampler(params) if self._device_sampling and device_samplable(params) else None
        smpl = None if dev is not None or (params.greedy and params.dry_multiplier <= 0) else \
            make_sampler(params, self.hp.n_vocab, self.hp.n_ctx_train, getattr(self, "token_table", None))
        st = RequestState(rid, params, smpl, len(prompt), t_submit=time.time(), dev=dev)
        if st.sampler is not None:
            for t in prompt[-params.repeat_last_n:]:
                st.sampler.accept(t)
        self.requests[rid] = st
        self.sched.add(rid, prompt, params.max_tokens, params.ignore_eos, getattr(params, "n_keep", None))
        return rid

    def cancel(self, req_id: int) -> bool:
        ok = self.sched.cancel(req_id)
        self._drain_events()
        return ok

    def has_work(self) -> bool:
        return not self.sched.idle() or self._inflight is not None

    # ------------------------------------------------------------------------------------------
    def _batch_views(self, n_tokens: int, n_seqs: int, n_out: int, max_q_len: int) -> ForwardBatch:
        d = self.io.d
        meta = None
        if max_q_len > 1:
            # host-side totals of a prompt step (the scheduler wrote these arrays; no device read): sizes of the gathered
            # K / V buffers and of the attention grid of the per-head prefill form
            h = self.io.h
            qs = h["q_start"][:n_seqs + 1]
            q_len, s_len = np.diff(qs), h["seq_lens"][:n_seqs]
            # kv_decode: cached rows of the sequences that only decode in this step (the per-head form would expand them all)
            meta = {"total_kv": int(s_len.sum()), "n_q_tiles": int(((q_len + 127) // 128).sum()),
                    "kv_decode": int(s_len[q_len <= 1].sum())}
        return ForwardBatch(tokens=d["tokens"][:n_tokens], positions=d["positions"][:n_tokens],
                            slot_mapping=d["slot_mapping"][:n_tokens],
                            block_tables=d["block_tables"].view(self.io.cap_seqs, self.max_blocks)[:n_seqs],
                            seq_lens=d["seq_lens"][:n_seqs], q_start=d["q_start"][:n_seqs + 1],
                            out_rows=d["out_rows"][:n_out], max_q_len=max_q_len, attn_meta=meta)

    def _sample_device(self, logits: torch.Tensor, mode: str) -> torch.Tensor:
        """Returns an int32 tensor: [n] token ids (greedy) or [n, 2k] (k float bit patterns + k ids)."""
        if mode == "greedy":
            return ops.argmax(logits)
        k = min(self.cfg.presample_count, logits.shape[-1])
        v, i = ops.topk_logits(logits, k)
        if mode == "sample":             # truncation, temperature and the draw on the device: only the id comes back
            n = logits.shape[0]
            rows = self.io.d["samp"].view(torch.float32).view(-1, 5)[:n]
            return ops.sample_topk(v.contiguous(), i.contiguous(), rows)
        if mode == "topk_lp":            # candidates plus the row's log-normaliser: log-probabilities on the host
            lse = torch.logsumexp(logits.float(), dim=-1, keepdim=True)
            return torch.cat([v.contiguous().view(torch.int32), i, lse.contiguous().view(torch.int32)], dim=-1)
        return torch.cat([v.contiguous().view(torch.int32), i], dim=-1)

    def _step_mode(self, states) -> str:
        """greedy: ids by arg-max; sample: at least one request is sampled on the device, none needs the host chain;
        topk: candidates go to the host chain."""
        if any(s.params.logprobs for s in states):
            return "topk_lp"
        if any(s.sampler is not None for s in states):
            return "topk"
        return "sample" if any(s.dev is not None for s in states) else "greedy"

    def _fill_sampling_rows(self, states, n_rows: int) -> list:
        """One (temperature, top_k, top_p, min_p, u) row per output row into the step's host buffer (temperature 0 = take
        the best candidate, for greedy requests and padding rows).  Returns the rows of device-sampled requests."""
        buf = self.io.h["samp"].view(np.float32).reshape(-1, 5)
        buf[:n_rows] = 0.0
        rows = []
        for i, st in enumerate(states):
            r = st.dev.row() if st.dev is not None else None
            rows.append(r)
            if r is not None:
                buf[i] = r
        return rows

    def _forward_sample(self, batch: ForwardBatch, mode: str) -> torch.Tensor:
        if getattr(self.model, "split", False) and self.device.type == "cuda":
            logits = self.model.forward(batch, self.kv_cache)
            with torch.cuda.device(logits.device):
                return self._sample_device(logits, mode)
        logits = self.model.forward(batch, self.kv_cache)
        if self._poison and bool(torch.isnan(logits).any()):
            raise RuntimeError("NaN logits with poisoned free blocks: a sequence read a cache block it does not own")
        return self._sample_device(logits, mode)

    def _poison_freed(self) -> None:
        blocks = self.kv.take_freed()
        if blocks.size == 0:
            return
        bs = self.cfg.block_size
        for il in range(self.hp.n_layer):
            layer = self.kv_cache[il]
            rows = (torch.from_numpy(blocks.astype(np.int64)).to(layer.device)[:, None] * bs +
                    torch.arange(bs, device=layer.device)[None, :]).reshape(-1)
            layer[rows] = float("nan")
        self.stats["poisoned_blocks"] += int(blocks.size)

    def _graph_for(self, bucket: int, mode: str):
        key = (bucket, mode)
        if key in self._graphs:
            return self._graphs[key]
        batch = self._batch_views(bucket, bucket, bucket, 1)
        # warm-up on a side stream (allocations, lazy init), then capture
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._forward_sample(batch, mode)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        n0 = ops.nat().launch_count if not ops.force_torch() else 0
        with torch.cuda.graph(g):
            out = self._forward_sample(batch, mode)
        if not ops.force_torch():
            self.graph_launches[key] = ops.nat().launch_count - n0
        self._graphs[key] = (g, out)
        self._host_barrier()             # capture time differs per rank; re-align before the first replay
        return self._graphs[key]

    def _host_barrier(self):
        comm = getattr(self.model, "comm", None)
        if comm is not None and hasattr(comm, "host_barrier"):
            comm.host_barrier()
        elif self.dp:
            import torch.distributed as dist
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            dist.barrier()

    def _idle_forward(self):
        """This rank has no tokens in this step but must serve its experts to the others."""
        if self._idle_graph is not None:
            self._idle_graph.replay()
        else:
            self.model.forward(None, None)

    def reset(self) -> None:
        """Drop every request and all cached tokens (recovery after a failed step: the scheduler may have been left
        between planning and commit).  Weights, cache memory and captured graphs stay."""
        cfg = self.cfg
        self.kv = PagedKV(self.n_blocks, cfg.block_size, cfg.n_parallel)
        self.sched = Scheduler(self.kv, cfg.n_parallel, cfg.n_batch, self.n_ctx_slot, self.hp.eos_id, cfg.n_keep,
                               cfg.cont_batching)
        if cfg.mixed_prompt_budget > 0:
            self.sched.set_mixed_prompt_budget(cfg.mixed_prompt_budget)
        self.requests.clear()
        self._pressure = False
        self._inflight = None
        if self._poison:
            self.kv.track_freed(True)
        self.stats["resets"] = self.stats.get("resets", 0) + 1

    def run_until_all_idle(self, max_steps: int = 1 << 30) -> int:
        """Data-parallel serving loop: step until no rank has work left.  Every rank leaves at the same step."""
        n = 0
        while n < max_steps:
            self.step()
            n += 1
            if not self.dp and not self.has_work():
                break
            if self.dp and self.dp_active == 0:
                break
        return n

    def warmup(self, modes: Iterable[str] = ("greedy",)):
        """Capture the decode graphs up front (the reference compiles its GE graph at context creation)."""
        if not self._use_graphs:
            return
        if self._device_sampling and "sample" not in modes:
            modes = tuple(modes) + ("sample",)      # requests sampled on the device replay their own graphs
        h = self.io.h
        h["samp"][:] = 0
        h["slot_mapping"][:] = -1
        h["seq_lens"][:] = 0
        h["q_start"][:] = np.arange(len(h["q_start"]))
        h["out_rows"][:] = np.arange(len(h["out_rows"]))
        self.io.upload()
        for b in self.cfg.graph_buckets:
            if b <= self.io.cap_seqs:
                for m in modes:
                    self._graph_for(b, m)
        if self.dp and self._idle_graph is None:
            # every rank runs the same sequence here (two warm-up passes, one capture), so the collectives pair up
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                for _ in range(2):
                    self.model.forward(None, None)
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.model.forward(None, None)
            self._idle_graph = g
            self._host_barrier()

    # ------------------------------------------------------------------------------------------
    def _maybe_defrag(self):
        if self.cfg.defrag_thold < 0 or self.kv.fragmentation() <= self.cfg.defrag_thold:
            return
        self.defrag(self.cfg.defrag_max_moves)

    def defrag(self, max_moves: int) -> int:
        src, dst = self.kv.defrag(max_moves)
        if len(src):
            self._copy_blocks(src, dst)
            self.stats["defrag_moves"] += len(src)
        return len(src)

    def _copy_blocks(self, src: np.ndarray, dst: np.ndarray):
        if isinstance(self.kv_cache, SplitCache):
            self.kv_cache.copy_blocks(src, dst)
            return
        s = torch.from_numpy(np.ascontiguousarray(src)).to(self.device)
        d = torch.from_numpy(np.ascontiguousarray(dst)).to(self.device)
        ops.kv_block_copy(self.kv_cache, s, d, self.cfg.block_size)

    def _drain_events(self) -> List[Tuple[int, int, Optional[str]]]:
        out = []
        for rid, slot, tok, fin, n_prompt, n_dec in self.sched.take_events():
            st = self.requests.get(rid)
            if st is None:
                continue
            if tok >= 0:
                st.output.append(tok)
                if len(st.output) == 1:
                    st.t_first = time.time()
                    if slot >= 0:
                        st.n_cached = self.sched.slot_cached(slot)
            if fin is not None:
                st.finish_reason = fin
                st.t_done = time.time()
            out.append((rid, tok, fin))
        return out

    def step(self) -> List[Tuple[int, int, Optional[str]]]:
        """Runs one engine step. Returns [(req_id, new_token, finish_reason_or_None)]."""
        if self._run_ahead:
            return self._step_ahead()
        return self._step_sync()

    # ---- running one step ahead (opt-in) -----------------------------------------------------------------------------
    # With greedy sampling on the device, the ids a step produces are the next step's input tokens: they can stay on the
    # device.  The engine then launches decode step k + 1 (its token buffer filled by a device copy from step k's output)
    # before it reads step k's ids, so the host's share of a step -- scheduling, packing, the upload, the graph launch and
    # the read-back -- overlaps the device's.  Events reach the caller one step later.  What cannot be known without the
    # ids is the end-of-sequence token: a sequence that produced it has by then been fed one token too many; that
    # output is dropped (Scheduler::resolve).  Whenever the next step is not a pure decode step of the same sequences
    # (a waiting request, a prompt chunk, scarce blocks, a sampler that needs the host), the engine first reads the ids
    # and continues synchronously.
    def set_run_ahead(self, on: bool) -> bool:
        """Switches run-ahead stepping on or off (tools that time single steps need the synchronous form); a step still in
        flight is completed first.  Returns the previous setting."""
        prev = self._run_ahead
        if self._inflight is not None:
            self.sched.commit(self._collect(self._inflight), self._inflight.n_out)
            self._inflight = None
        self._run_ahead = bool(on) and not self.dp and not getattr(self.model, "split", False)
        if self._run_ahead and len(self._out_hosts) < 2:
            extra = torch.zeros_like(self._out_host)
            self._out_hosts.append(extra.pin_memory() if self.device.type == "cuda" else extra)
        return prev

    def _all_greedy(self) -> bool:
        """No live request needs the host sampler chain (ids are chosen on the device: arg-max or the device sampler)."""
        return all(st.sampler is None and not st.params.logprobs for st in self.requests.values() if st.finish_reason is None)

    def _check_device_status(self, host: Optional[torch.Tensor]) -> None:
        """``host``: the pinned copy of the status words taken behind a step, valid once that step's stream work is done."""
        if host is None or int(host[0]) == 0:
            return
        st = host.tolist()
        ws = ops.nat().workspace(self.device)
        ws.status.zero_()
        ws.counters.zero_()
        ws.route_counter.zero_()
        host.zero_()
        self.stats["device_faults"] = self.stats.get("device_faults", 0) + 1
        names = {1: "wait timeout", 2: "index out of bounds", 3: "misaligned"}
        raise RuntimeError(f"kernel status: {names.get(st[0], st[0])} at site {st[1]} block {st[2]} extra {st[3]}: step discarded")

    def _collect(self, infl: _InFlight) -> np.ndarray:
        if infl.event is not None:
            infl.event.synchronize()
        self._check_device_status(infl.status)
        self.stats["d2h_bytes"] += infl.n_out * 4 + (16 if infl.status is not None else 0)
        return infl.host[:infl.n_out].numpy().astype(np.int32, copy=True)

    def _launch_greedy(self, n_tokens: int, n_seqs: int, n_out: int, max_q: int, feedback: Optional[_InFlight]) -> _InFlight:
        """Launches a step whose ids are chosen on the device (arg-max, or the device sampler for requests that use it)."""
        io = self.io
        states = [self.requests[int(r)] for r in self.sched.out_reqs(n_out)]
        mode = self._step_mode(states)
        if mode == "sample":
            self._fill_sampling_rows(states, io.cap_seqs)
        use_graph = self._use_graphs and max_q == 1 and n_seqs == n_tokens and n_seqs <= max(self.cfg.graph_buckets) \
            and getattr(self.model, "tensor_hook", None) is None
        bucket = next(b for b in self.cfg.graph_buckets if b >= n_seqs) if use_graph else 0
        if use_graph and bucket > n_seqs:
            h = io.h
            h["tokens"][n_seqs:bucket] = 0
            h["positions"][n_seqs:bucket] = 0
            h["slot_mapping"][n_seqs:bucket] = -1
            h["seq_lens"][n_seqs:bucket] = 0
            h["q_start"][n_seqs:bucket + 1] = np.arange(n_seqs, bucket + 1)
            h["out_rows"][n_out:bucket] = np.arange(n_out, bucket)
            h["block_tables"][n_seqs * self.max_blocks: bucket * self.max_blocks] = 0
        io.upload()
        if feedback is not None:
            # this step's tokens are the ids the step in flight sampled: a device-to-device copy, in output-row order
            row_of = {int(sl): i for i, sl in enumerate(feedback.out_slots)}
            src = np.fromiter((row_of[int(sl)] for sl in io.h["seq_slots"][:n_seqs]), dtype=np.int64, count=n_seqs)
            prev = feedback.out.reshape(-1)
            if np.array_equal(src, np.arange(n_seqs)):
                io.d["tokens"][:n_seqs].copy_(prev[:n_seqs])
            else:
                io.d["tokens"][:n_seqs].copy_(prev.index_select(0, torch.from_numpy(src).to(prev.device)))
        if use_graph:
            g, out = self._graph_for(bucket, mode)
            g.replay()
            self.launches += self.graph_launches.get((bucket, mode), 0)
            self.stats["graph_steps"] += 1
        else:
            batch = self._batch_views(n_tokens, n_seqs, n_out, max_q)
            n0 = ops.nat().launch_count if self.device.type == "cuda" and not ops.force_torch() else 0
            out = self._forward_sample(batch, mode)
            if self.device.type == "cuda" and not ops.force_torch():
                self.launches += ops.nat().launch_count - n0
            self.stats["eager_steps"] += 1
        host = self._out_hosts[self._flip]
        self._flip ^= 1
        host[:n_out].copy_(out.reshape(-1)[:n_out], non_blocking=True)
        status = None
        if self._status_hosts is not None:
            status = self._status_hosts[self._flip]
            status.copy_(self._status_dev, non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        self.stats["steps"] += 1
        self.stats["tokens_in"] += n_tokens
        self.stats["tokens_out"] += n_out
        self.stats["h2d_bytes"] += io.h2d_bytes
        return _InFlight(out, host, event, n_out, io.h["out_slots"][:n_out].copy(), status)

    def _trace_ahead(self, pt, ev, launched, n_tokens=0, n_seqs=0, n_out=0, max_q=0) -> None:
        """Step trace of the run-ahead path: "step" for a call that launched one (its events belong to the step before),
        "collect" for a call that only read the ids of the step in flight."""
        if pt is None:
            return
        pt.mark("finish")
        common = dict(kv_used=self.kv.used_blocks, kv_total=self.n_blocks, waiting=self.sched.n_waiting(),
                      running=self.sched.n_running(), finished=sum(1 for e in ev if e[2] is not None), phase_ms=pt.ms)
        if launched:
            self.tracer.emit("step", step=self.stats["steps"], tokens=n_tokens, seqs=n_seqs, outputs=n_out, max_q=max_q,
                             mode="ahead", frag=round(self.kv.fragmentation(), 4), **common)
        else:
            self.tracer.emit("collect", **common)

    @torch.no_grad()
    def _step_ahead(self) -> List[Tuple[int, int, Optional[str]]]:
        io, infl = self.io, self._inflight
        pt = PhaseTimer() if self.tracer.enabled else None
        usable = self._all_greedy() and not self._poison and not fault.armed("kv_alloc") and not fault.armed("engine_step")
        if not usable:                       # finish what is in flight, then step the ordinary way (its events are queued)
            if infl is not None:
                self.sched.commit(self._collect(infl), infl.n_out)
                self._inflight = None
            return self._step_sync()
        if infl is not None:
            if self.sched.can_run_ahead():
                self.sched.commit_deferred(infl.n_out)
                self._stage ^= 1
                io.use_stage(self._stage)
                info = self.sched.step(io.arrays)
                n_tokens, n_seqs, n_out, _, max_q, _, n_copies = (int(x) for x in info[:7])
                if pt:
                    pt.mark("schedule")
                nxt = None
                if n_tokens > 0:
                    if n_copies:
                        src, dst = self.kv.take_copies()
                        self._copy_blocks(src, dst)
                    nxt = self._launch_greedy(n_tokens, n_seqs, n_out, max_q, infl)
                    self.stats["run_ahead_steps"] = self.stats.get("run_ahead_steps", 0) + 1
                if pt:
                    pt.mark("launch")
                self.sched.resolve(self._collect(infl), infl.n_out)
                self._inflight = nxt
                if pt:
                    pt.mark("wait")
                ev = self._drain_events()
                self._maybe_defrag()
                self._trace_ahead(pt, ev, nxt is not None, n_tokens, n_seqs, n_out, max_q)
                return ev
            self.sched.commit(self._collect(infl), infl.n_out)
            self._inflight = None
            ev = self._drain_events()
            self._maybe_defrag()
            self._trace_ahead(pt, ev, False)
            return ev
        self._stage ^= 1
        io.use_stage(self._stage)
        info = self.sched.step(io.arrays)
        n_tokens, n_seqs, n_out, _, max_q, _, n_copies = (int(x) for x in info[:7])
        if n_tokens == 0:
            return self._drain_events()
        if pt:
            pt.mark("schedule")
        if n_copies:
            src, dst = self.kv.take_copies()
            self._copy_blocks(src, dst)
        if n_out == 0:                       # a prompt chunk without an output row: nothing to wait for
            io.upload()
            self.model.forward(self._batch_views(n_tokens, n_seqs, 0, max_q), self.kv_cache)
            self.stats["steps"] += 1
            self.stats["eager_steps"] += 1
            self.stats["tokens_in"] += n_tokens
            self.stats["h2d_bytes"] += io.h2d_bytes
            self.sched.commit(np.empty(0, dtype=np.int32), 0)
        else:
            self._inflight = self._launch_greedy(n_tokens, n_seqs, n_out, max_q, None)
        if pt:
            pt.mark("launch")
        ev = self._drain_events()
        self._maybe_defrag()
        self._trace_ahead(pt, ev, True, n_tokens, n_seqs, n_out, max_q)
        return ev

    @torch.no_grad()
    def _step_sync(self) -> List[Tuple[int, int, Optional[str]]]:
        io = self.io
        fault.check("engine_step")
        if self._pressure:
            self.kv.unreserve()
            self._pressure = False
        if fault.armed("kv_alloc") and fault.hit("kv_alloc"):
            self.kv.reserve(self.kv.n_blocks)          # this step sees an allocator without free blocks
            self._pressure = True
        pt = PhaseTimer() if self.tracer.enabled else None
        info = self.sched.step(io.arrays)
        n_tokens, n_seqs, n_out, n_dec, max_q, _, n_copies = (int(x) for x in info[:7])
        if pt:
            pt.mark("schedule")
        if self.dp:
            import torch.distributed as dist
            self._dp_flag.fill_(1 if (n_tokens > 0 or self.has_work()) else 0)
            dist.all_reduce(self._dp_flag)
        if n_tokens == 0:
            if self.dp:
                self._idle_forward()
                self.dp_active = int(self._dp_flag.item())
                self.stats["idle_steps"] = self.stats.get("idle_steps", 0) + 1
            return self._drain_events()
        if n_copies:
            src, dst = self.kv.take_copies()
            self._copy_blocks(src, dst)
        if self._poison:
            self._poison_freed()             # after the copies: a block may be freed while a copy out of it is still queued
        states = [self.requests[int(r)] for r in self.sched.out_reqs(n_out)] if n_out else []
        mode = self._step_mode(states)
        samp_rows = self._fill_sampling_rows(states, io.cap_seqs) if mode != "greedy" else None
        use_graph = self._use_graphs and max_q == 1 and n_seqs == n_tokens and n_seqs <= max(self.cfg.graph_buckets) \
            and getattr(self.model, "tensor_hook", None) is None
        if use_graph and self.dp:
            # ranks capture in lockstep during warmup() only: a capture on first use would run collectives alone
            use_graph = (next(b for b in self.cfg.graph_buckets if b >= n_seqs), mode) in self._graphs
        if use_graph:
            bucket = next(b for b in self.cfg.graph_buckets if b >= n_seqs)
            h = io.h
            if bucket > n_seqs:
                h["tokens"][n_seqs:bucket] = 0
                h["positions"][n_seqs:bucket] = 0
                h["slot_mapping"][n_seqs:bucket] = -1
                h["seq_lens"][n_seqs:bucket] = 0
                h["q_start"][n_seqs:bucket + 1] = np.arange(n_seqs, bucket + 1)
                h["out_rows"][n_out:bucket] = np.arange(n_out, bucket)
                h["block_tables"][n_seqs * self.max_blocks: bucket * self.max_blocks] = 0
            io.upload()                      # before a first-use capture too: its warm-up runs read these buffers
            g, out = self._graph_for(bucket, mode)
            g.replay()
            self.launches += self.graph_launches.get((bucket, mode), 0)
            self.stats["graph_steps"] += 1
        else:
            io.upload()
            batch = self._batch_views(n_tokens, n_seqs, n_out, max_q)
            n0 = ops.nat().launch_count if self.device.type == "cuda" and not ops.force_torch() else 0
            out = self._forward_sample(batch, mode) if n_out else None
            if n_out == 0:
                self.model.forward(batch, self.kv_cache)
            if self.device.type == "cuda" and not ops.force_torch():
                self.launches += ops.nat().launch_count - n0
            self.stats["eager_steps"] += 1
        if pt:
            pt.mark("launch")
        self.stats["steps"] += 1
        self.stats["tokens_in"] += n_tokens
        self.stats["h2d_bytes"] += io.h2d_bytes
        if n_out:
            flat = out.reshape(-1)
            n_el = flat.numel()
            host = self._out_host[:n_el]
            host.copy_(flat, non_blocking=True)
            if self._status_hosts is not None:
                self._status_hosts[0].copy_(self._status_dev, non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream(out.device).synchronize()
            self._check_device_status(self._status_hosts[0] if self._status_hosts is not None else None)
            if pt:
                pt.mark("wait")
            self.stats["d2h_bytes"] += n_el * 4 + (16 if self._status_hosts is not None else 0)
            res = host.numpy().reshape(out.shape[0], -1)
            sampled = np.empty(n_out, dtype=np.int32)
            if mode in ("greedy", "sample"):
                sampled[:] = res[:n_out, 0]
            else:
                k = res.shape[1] // 2
                for i, st in enumerate(states):
                    vals = res[i, :k].view(np.float32)
                    ids = res[i, k:2 * k]
                    if st.dev is not None:
                        sampled[i] = st.dev.sample_host(vals, ids, samp_rows[i])
                    elif st.sampler is None:
                        sampled[i] = ids[int(np.argmax(vals))]
                    else:
                        sampled[i] = st.sampler.sample(vals, ids)
                    if mode == "topk_lp" and st.params.logprobs:
                        lp = vals.astype(np.float64) - float(res[i, 2 * k:2 * k + 1].view(np.float32)[0])
                        hit = np.nonzero(ids == sampled[i])[0]
                        n_alt = max(0, min(int(st.params.top_logprobs), k))
                        st.logprobs.append((int(sampled[i]), float(lp[hit[0]]) if hit.size else float("-inf"),
                                            [(int(ids[j]), float(lp[j])) for j in range(n_alt)]))
            for i, st in enumerate(states):
                if st.sampler is not None:
                    st.sampler.accept(int(sampled[i]))
            self.sched.commit(sampled, n_out)
            self.stats["tokens_out"] += n_out
        else:
            self.sched.commit(np.empty(0, dtype=np.int32), 0)
        if self.dp:
            self.dp_active = int(self._dp_flag.item())
        ev = self._drain_events()
        self._maybe_defrag()
        if pt:
            pt.mark("finish")
            self.tracer.emit("step", step=self.stats["steps"], tokens=n_tokens, seqs=n_seqs, outputs=n_out, max_q=max_q,
                             mode="graph" if use_graph else "eager", kv_used=self.kv.used_blocks, kv_total=self.n_blocks,
                             frag=round(self.kv.fragmentation(), 4), waiting=self.sched.n_waiting(), running=self.sched.n_running(),
                             finished=sum(1 for e in ev if e[2] is not None), phase_ms=pt.ms)
        return ev

    # ------------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None,
                 max_new_tokens: Optional[int] = None) -> List[List[int]]:
        """Blocking helper: run the given prompts to completion, return the generated ids per prompt."""
        ids = []
        for p in prompts:
            sp = params or SamplingParams()
            if max_new_tokens is not None:
                sp = SamplingParams(**{**sp.__dict__, "max_tokens": max_new_tokens})
            ids.append(self.add_request(p, sp))
        if self.dp:
            self.run_until_all_idle()
        while self.has_work():
            self.step()
        outs = [self.requests[i].output for i in ids]
        for i in ids:
            self.requests.pop(i, None)
        return outs
