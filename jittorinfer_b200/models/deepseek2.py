"""DeepSeek-V2 / V2-Lite module graph over a paged compressed-latent KV cache.

This replaces the reference's per-step ggml graph construction (``llm_build_deepseek2``,
src/llama-graph-deepseek2.cpp:113-405, with sub-graphs in src/llama-graph-attn.cpp and
src/llama-graph-ffn.cpp) by a fixed PyTorch module graph whose ops are the sm_100a kernels in
``jittorinfer_b200.ops``; the engine replays it as CUDA graphs per decode bucket.

Differences from the reference that are deliberate:

* attention always runs in the weight-absorbed MLA form over one latent row ``[c_kv | k_pe]``
  per token (the reference also keeps a transposed duplicate of ``c_kv``,
  src/llama-graph-attn.cpp:233-255, and its shipped multi-card server uses per-head K/V);
* ``attn_q``/``attn_q_a`` and ``attn_kv_a_mqa`` share their input, so they are one GEMM;
* sequence lengths and block tables replace the O(T*S) host-built mask
  (src/llama-context.cpp:326-423);
* the q-LoRA branch is selected by ``q_lora_rank``, not by ``n_layer == 27``.

Under tensor parallelism every rank holds the full residual stream; attention heads, dense/shared
FFN columns and routed experts are sharded (see ``models.weights.shard_dim``) and the two partial
sums per layer are combined by ``comm.all_reduce`` (reference: src/llama-graph-deepseek2.cpp:294-297,
365-368) or by the fused GEMM+all-reduce kernel when the communicator provides one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import ops
from ..utils import trace as _trace
from .hparams import DeepSeek2HParams
from .weights import ShardSpec


@dataclass
class ForwardBatch:
    """One engine step's inputs (all device tensors, int32 unless noted).

    ``tokens/positions/slot_mapping`` have one entry per query token; tokens of one sequence are
    contiguous.  Sequence ``b`` owns rows ``q_start[b]:q_start[b+1]`` and, after this step, has
    ``seq_lens[b]`` cached tokens.  ``slot_mapping[i] < 0`` marks a padding row.
    ``out_rows`` selects the rows whose logits are wanted.
    """
    tokens: torch.Tensor
    positions: torch.Tensor
    slot_mapping: torch.Tensor
    block_tables: torch.Tensor
    seq_lens: torch.Tensor
    q_start: torch.Tensor
    out_rows: torch.Tensor
    max_q_len: int = 1
    attn_meta: Optional[object] = None


def _batch_to(b: ForwardBatch, dev: torch.device) -> ForwardBatch:
    mv = lambda t: None if t is None else t.to(dev, non_blocking=True)
    return ForwardBatch(mv(b.tokens), mv(b.positions), mv(b.slot_mapping), mv(b.block_tables), mv(b.seq_lens), mv(b.q_start),
                        mv(b.out_rows), b.max_q_len, None)


def assign_layers(n_layer: int, devices, tensor_split=None):
    """Contiguous layer ranges per device, proportional to ``tensor_split`` (even when omitted), every device getting
    at least one layer when there are enough (reference: src/llama-model.cpp:495-540, 551-563)."""
    devices = list(devices)
    n = len(devices)
    w = [float(x) for x in tensor_split][:n] if tensor_split else [1.0] * n
    w += [0.0] * (n - len(w))
    total = sum(w) or 1.0
    bounds, acc = [], 0.0
    for x in w:
        acc += x
        bounds.append(acc / total)
    out = []
    for il in range(n_layer):
        frac = (il + 0.5) / n_layer
        out.append(devices[next(i for i, b in enumerate(bounds) if frac <= b + 1e-9)])
    return out


class _Layer:
    __slots__ = ("attn_norm", "w_qkv_a", "q_a_norm", "w_q_b", "kv_a_norm", "w_uk", "w_uv", "w_kv_b", "w_o", "ffn_norm",
                 "w_gate", "w_up", "w_down", "w_router", "router_bias", "w_gate_exps", "w_up_exps", "w_down_exps",
                 "w_gate_sh", "w_up_sh", "w_down_sh", "is_moe", "n_shared_merged")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


class DeepSeek2Model:
    def __init__(self, hp: DeepSeek2HParams, weights: Iterable[Tuple[str, torch.Tensor]],
                 dtype: torch.dtype = torch.bfloat16, device="cpu", spec: ShardSpec = ShardSpec(),
                 comm=None, max_positions: int = 8192, block_size: int = 64, ep=None, layer_devices=None):
        self.hp = hp
        self.dtype = dtype
        self.device = torch.device(device)
        self.spec = spec
        self.comm = comm
        # Layer split (the reference's default LLAMA_SPLIT_MODE_LAYER, src/llama-model.cpp:495-540): consecutive layer
        # ranges live on consecutive devices of this one process and the activations hop between them; no pipelining
        # (the reference's scheduler cannot pipeline on its device back end either, ggml-cann.cpp:2301-2306).
        self.layer_dev = [torch.device(d) for d in layer_devices] if layer_devices else [self.device] * hp.n_layer
        if len(self.layer_dev) != hp.n_layer:
            raise ValueError("layer_devices needs one entry per layer")
        self.split = any(d != self.device for d in self.layer_dev)
        if self.split and spec.sharded:
            raise ValueError("layer split and tensor / expert parallelism are separate modes")
        self.out_device = self.layer_dev[-1]
        self._cur_dev = self.device
        self._uploaders = {}
        # Debug tap, the counterpart of the reference's per-node eval callback (cb_eval, include/llama.h:563-564;
        # ggml/src/ggml-backend.cpp:1543-1580): when set, called as tensor_hook(name, tensor) with the block outputs of
        # every layer ("blk.3.attn_out", "blk.3.ffn_inp", "blk.3.ffn_out") and "result_norm" / "result_output".  The engine
        # runs eagerly while a hook is installed (a hook cannot run inside a captured graph).
        self.tensor_hook = None
        self.ep = ep                      # all-to-all dispatcher (data-parallel attention + expert parallelism)
        self.block_size = block_size
        if spec.dp_attention:
            if ep is None and spec.sharded:
                raise ValueError("dp_attention needs an expert-parallel dispatcher (ep=...)")
            self.n_head_local = hp.n_head
        else:
            if hp.n_head % spec.tp_size:
                raise ValueError("n_head must be divisible by tp_size")
            self.n_head_local = hp.n_head // spec.tp_size
        if spec.expert_parallel or spec.dp_attention:
            if hp.n_expert % spec.tp_size:
                raise ValueError("n_expert must be divisible by the expert-parallel size")
            self.n_expert_local = hp.n_expert // spec.tp_size
            self.expert_base = spec.tp_rank * self.n_expert_local
        else:
            self.n_expert_local = hp.n_expert
            self.expert_base = 0
        self.layers: List[_Layer] = [_Layer() for _ in range(hp.n_layer)]
        self.tok_embd = None
        self.out_norm = None
        self.w_out = None
        self._load(weights)
        lo, hi = hp.yarn_corr_dims()
        self.max_positions = max_positions
        self.rope_table = ops.ref.yarn_table(max_positions, hp.qk_rope_head_dim, hp.rope_freq_base, hp.freq_scale,
                                             hp.ext_factor, hp.rope_attn, lo, hi, device=self.device)
        self._rope_by_dev = {}

    def _rope(self, dev: torch.device) -> torch.Tensor:
        if not self.split or dev == self.rope_table.device:
            return self.rope_table
        t = self._rope_by_dev.get(dev)
        if t is None or t.shape != self.rope_table.shape:
            t = self._rope_by_dev[dev] = self.rope_table.to(dev)
        return t

    # ---- weight intake -------------------------------------------------------------------
    def _dev(self, t: torch.Tensor, dtype=None) -> torch.Tensor:
        if t.device.type == "cpu" and self._cur_dev.type == "cuda" and t.numel() * t.element_size() >= (256 << 20):
            up = self._uploaders.get(self._cur_dev)
            if up is None:
                from .weights import StagedUploader
                up = self._uploaders[self._cur_dev] = StagedUploader(self._cur_dev)
            return up.upload(t, dtype or self.dtype)          # large tensors go through pinned staging buffers
        return t.to(device=self._cur_dev, dtype=dtype or self.dtype).contiguous()

    def _load(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        hp = self.hp
        H, dn, dv, r = self.n_head_local, hp.qk_nope_head_dim, hp.v_head_dim, hp.kv_lora_rank
        pend: Dict[str, torch.Tensor] = {}
        for name, t in weights:
            _trace.log_tensor(name, t.shape, t.dtype, f"rank {self.spec.tp_rank}/{self.spec.tp_size}" if self.spec.sharded else "")
            if name.startswith("blk."):
                self._cur_dev = self.layer_dev[int(name.split(".", 2)[1])]
            else:
                self._cur_dev = self.out_device if name in ("output_norm.weight", "output.weight") else self.device
            if name == "token_embd.weight":
                self.tok_embd = self._dev(t)
            elif name == "output_norm.weight":
                self.out_norm = self._dev(t, torch.float32)
            elif name == "output.weight":
                self.w_out = self._dev(t)
            elif name.startswith("blk."):
                _, il, base, _ = name.split(".", 3)
                L = self.layers[int(il)]
                key = f"{il}.{base}"
                if base == "attn_norm":
                    L.attn_norm = self._dev(t, torch.float32)
                elif base == "ffn_norm":
                    L.ffn_norm = self._dev(t, torch.float32)
                elif base == "attn_q_a_norm":
                    L.q_a_norm = self._dev(t, torch.float32)
                elif base == "attn_kv_a_norm":
                    L.kv_a_norm = self._dev(t, torch.float32)
                elif base in ("attn_q", "attn_q_a", "attn_kv_a_mqa"):
                    pend[key] = self._dev(t)
                    qk = f"{il}.attn_q" if hp.is_lite else f"{il}.attn_q_a"
                    kk = f"{il}.attn_kv_a_mqa"
                    if qk in pend and kk in pend:
                        L.w_qkv_a = torch.cat([pend.pop(qk), pend.pop(kk)], dim=0).contiguous()
                elif base == "attn_q_b":
                    L.w_q_b = self._dev(t)
                elif base == "attn_kv_b":
                    # load-time re-layout into the absorbed factors (reference: wkv_b_post_process,
                    # src/llama-model.cpp:408-459)
                    w = self._dev(t).view(H, dn + dv, r)
                    L.w_uk = w[:, :dn, :].transpose(1, 2).contiguous()   # [H, r, dn]: q_abs = q_nope @ w_uk[h]^T
                    L.w_uv = w[:, dn:, :].contiguous()                   # [H, dv, r]: o = o_lat @ w_uv[h]^T
                    L.w_kv_b = w.reshape(H * (dn + dv), r)               # as stored: prompt chunks expand k_nope | v per head
                elif base == "attn_output":
                    L.w_o = self._dev(t)
                elif base == "ffn_gate":
                    L.w_gate = self._dev(t)
                elif base == "ffn_up":
                    L.w_up = self._dev(t)
                elif base == "ffn_down":
                    L.w_down = self._dev(t)
                elif base == "ffn_gate_inp":
                    L.w_router = self._dev(t, torch.float32)
                    L.is_moe = True
                elif base == "exp_probs_b":
                    L.router_bias = self._dev(t, torch.float32)
                elif base == "ffn_gate_exps":
                    L.w_gate_exps = self._dev(t)
                elif base == "ffn_up_exps":
                    L.w_up_exps = self._dev(t)
                elif base == "ffn_down_exps":
                    L.w_down_exps = self._dev(t)
                elif base == "ffn_gate_shexp":
                    L.w_gate_sh = self._dev(t)
                elif base == "ffn_up_shexp":
                    L.w_up_sh = self._dev(t)
                elif base == "ffn_down_shexp":
                    L.w_down_sh = self._dev(t)
                else:
                    raise KeyError(f"unknown tensor {name}")
            else:
                raise KeyError(f"unknown tensor {name}")
        self._cur_dev = self.device
        self._uploaders.clear()               # release the pinned staging buffers
        if self.w_out is None:
            self.w_out = self.tok_embd if self.out_device == self.device else self.tok_embd.to(self.out_device)
        if not self.spec.sharded or not (self.spec.expert_parallel or self.spec.dp_attention):
            # single GPU, or every expert's FFN columns sharded over the ranks: the (local part of the) shared experts has
            # the (local) routed experts' shape, so it becomes experts E, E+1, ... of the grouped GEMMs (two fewer launches
            # per layer, better fill); the router appends them to every token.  Any split of the shared FFN's hidden units
            # into groups of the local expert width is a valid set of experts: the block is a sum over hidden units.
            for L in self.layers:
                L.n_shared_merged = 0
                F = L.w_gate_exps.shape[1] if L.is_moe and L.w_gate_exps is not None else hp.n_ff_exp
                if L.is_moe and L.w_gate_sh is not None and L.w_gate_sh.shape[0] % F == 0:
                    ns, d = L.w_gate_sh.shape[0] // F, hp.n_embd
                    L.w_gate_exps = torch.cat([L.w_gate_exps, L.w_gate_sh.view(ns, F, d)], dim=0)
                    L.w_up_exps = torch.cat([L.w_up_exps, L.w_up_sh.view(ns, F, d)], dim=0)
                    L.w_down_exps = torch.cat([L.w_down_exps, L.w_down_sh.view(d, ns, F).permute(1, 0, 2).contiguous()], dim=0)
                    L.w_gate_sh = L.w_up_sh = L.w_down_sh = None
                    L.n_shared_merged = ns
        for il, L in enumerate(self.layers):
            need = ["attn_norm", "w_qkv_a", "kv_a_norm", "w_uk", "w_o", "ffn_norm"]
            need += ["w_router", "w_gate_exps", "w_up_exps", "w_down_exps"] if L.is_moe else ["w_gate", "w_up", "w_down"]
            missing = [n for n in need if getattr(L, n) is None]
            if missing:
                raise ValueError(f"layer {il}: missing tensors {missing}")

    def weight_bytes(self) -> int:
        n = 0
        seen = set()
        for obj in [self] + self.layers:
            names = obj.__slots__ if hasattr(obj, "__slots__") else ("tok_embd", "out_norm", "w_out")
            for s in names:
                t = getattr(obj, s, None)
                if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    n += t.numel() * t.element_size()
        return n

    # ---- forward ---------------------------------------------------------------------------
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.comm is not None and self.spec.sharded:
            return self.comm.all_reduce(x)
        return x

    def _row_parallel(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """y = all_reduce(x_shard @ w_shard^T) + residual.  One fused kernel when the communicator has it."""
        if self.comm is not None and self.spec.sharded and not self.spec.dp_attention:
            return self.comm.linear_all_reduce(x, w, residual)
        return ops.linear(x, w, residual=residual)

    def _attention(self, L: _Layer, h: torch.Tensor, batch: ForwardBatch, cache_l: torch.Tensor) -> torch.Tensor:
        return self._attention_from_qkv(L, ops.linear(h, L.w_qkv_a), batch, cache_l)

    def _attention_from_qkv(self, L: _Layer, qkv: torch.Tensor, batch: ForwardBatch, cache_l: torch.Tensor) -> torch.Tensor:
        hp = self.hp
        H, dn, dr, r = self.n_head_local, hp.qk_nope_head_dim, hp.qk_rope_head_dim, hp.kv_lora_rank
        T = qkv.shape[0]
        h = qkv
        nq = qkv.shape[1] - hp.kv_row
        ckv = qkv[:, nq:]
        if hp.is_lite:
            q = qkv[:, :nq]
        else:
            qa, _ = ops.rmsnorm(qkv[:, :nq], L.q_a_norm, hp.rms_eps)
            q = ops.linear(qa, L.w_q_b)
        if batch.max_q_len > 1 and ops.use_native(q) and q.dtype == torch.bfloat16 and not self.split and \
                ops.nat().mha_prefill_ok(T, dn, dr, hp.v_head_dim, r, self.block_size, batch.attn_meta):
            # prompt chunk: per-head attention over K / V expanded from the latent rows (3.4x fewer FLOPs than the absorbed
            # form); the RoPE part of q is rotated in place, the latent row still goes to the cache for later decode steps
            ops.mla_qkv_post(q, ckv, L.kv_a_norm, hp.rms_eps, self._rope(h.device), batch.positions, batch.slot_mapping, cache_l, None,
                             H, dn, dr, r)
            return ops.nat().mha_prefill(q, cache_l, L.w_kv_b, batch.block_tables, batch.seq_lens, batch.q_start, hp.kq_scale, H,
                                         self.block_size, batch.attn_meta)
        q_full = torch.empty(T, H, r + dr, dtype=h.dtype, device=h.device)
        q_nope = ops.mla_qkv_post(q, ckv, L.kv_a_norm, hp.rms_eps, self._rope(h.device), batch.positions,
                                  batch.slot_mapping, cache_l, q_full, H, dn, dr, r)
        ops.q_absorb(q_nope, L.w_uk, q_full, r)
        o_lat = ops.mla_attention(q_full, cache_l, batch.block_tables, batch.seq_lens, batch.q_start, hp.kq_scale,
                                  r, self.block_size, batch.max_q_len, batch.attn_meta)
        return ops.v_up(o_lat, L.w_uv)

    def _mlp(self, L: _Layer, residual: torch.Tensor, norm=None):
        """The feed-forward block on ``residual`` (its input norm included): returns residual + ffn(rmsnorm(residual)).
        ``norm=(weight, eps)`` (MoE blocks): returns (x, rmsnorm(x) * weight), the next block's input norm."""
        hp = self.hp
        if not L.is_moe:
            g, _ = ops.rmsnorm(residual, L.ffn_norm, hp.rms_eps)
            hmid = ops.gateup_silu(g, L.w_gate, L.w_up)
            return self._row_parallel(hmid, L.w_down, residual)
        dp = self.spec.dp_attention and self.spec.sharded
        base = self.expert_base if self.spec.expert_parallel else 0
        # the router launch of a decode batch also normalises its input rows and sorts the pairs by local expert
        ids, wts, g = ops.moe_gate(residual, L.w_router, L.router_bias, hp.n_expert_used, hp.n_group, hp.topk_group,
                                   hp.expert_weights_scale, hp.expert_weights_norm, hp.expert_gating_func == "sigmoid",
                                   L.n_shared_merged or 0, hp.group_score_top2,
                                   route=None if dp else (base, L.w_gate_exps.shape[0]), pre_norm=(L.ffn_norm, hp.rms_eps))
        if dp:
            shared = None
            if L.w_gate_sh is not None:
                shared = ops.linear(ops.gateup_silu(g, L.w_gate_sh, L.w_up_sh), L.w_down_sh)
            return self.ep.moe_ffn(g, residual, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, shared)
        if self.comm is not None and self.spec.sharded:
            if getattr(self.comm, "fused_combine", False) and self.comm.fused and g.is_cuda and g.shape[0] <= self.comm.max_rows:
                # decode batches: combine, all-reduce, residual (and the next block's norm) in one launch
                return self.comm.moe_ffn_all_reduce(g, residual, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, L.w_gate_sh,
                                                    L.w_up_sh, L.w_down_sh, base, hp.n_expert, norm)
            part = ops.moe_ffn(g, None, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, L.w_gate_sh, L.w_up_sh,
                               L.w_down_sh, base, n_expert=hp.n_expert)
            return self.comm.all_reduce(part, residual)
        return ops.moe_ffn(g, residual, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, L.w_gate_sh, L.w_up_sh,
                           L.w_down_sh, base, n_expert=hp.n_expert, norm=norm)

    def _forward_sp(self, batch: ForwardBatch, kv_cache) -> torch.Tensor:
        """Tensor-parallel forward with a sequence-parallel residual stream (large prefill batches): every rank keeps
        R = ceil(T / N) token rows between the blocks; row-parallel GEMMs end in a reduce-scatter, column-parallel ones
        start from an all-gather.  Attention, routing and the experts still see all tokens (the latent cache is
        replicated and expert parallelism here replicates tokens), so only the norms, the residual adds and the
        collectives' second halves shrink -- and every row is reduced by exactly one rank."""
        hp, comm = self.hp, self.comm
        W, rk = self.spec.tp_size, self.spec.tp_rank
        T = batch.tokens.shape[0]
        R = (T + W - 1) // W
        Tp = R * W
        b = batch
        if Tp > T:       # pad with rows that belong to no sequence and write no cache slot
            pad = Tp - T
            z = torch.zeros(pad, dtype=batch.tokens.dtype, device=batch.tokens.device)
            b = ForwardBatch(torch.cat([batch.tokens, z]), torch.cat([batch.positions, z]),
                             torch.cat([batch.slot_mapping, torch.full_like(z, -1)]), batch.block_tables, batch.seq_lens,
                             batch.q_start, batch.out_rows, batch.max_q_len, None)
        x = ops.embed_gather(self.tok_embd, b.tokens)[rk * R:(rk + 1) * R].contiguous()
        for il, L in enumerate(self.layers):
            h_loc, _ = ops.rmsnorm(x, L.attn_norm, hp.rms_eps)
            qkv = comm.allgather_linear(h_loc, L.w_qkv_a)
            a = self._attention_from_qkv(L, qkv, b, kv_cache[il])
            if Tp > T:
                a[T:] = 0
            y = comm.linear_reduce_scatter(a, L.w_o, x)
            g_loc, _ = ops.rmsnorm(y, L.ffn_norm, hp.rms_eps)
            if not L.is_moe:
                hmid = comm.allgather_linear(g_loc, L.w_gate, L.w_up)
                x = comm.linear_reduce_scatter(hmid, L.w_down, y)
            else:
                g = comm.all_gather_rows(g_loc)
                ids, wts = ops.moe_gate(g, L.w_router, L.router_bias, hp.n_expert_used, hp.n_group, hp.topk_group,
                                        hp.expert_weights_scale, hp.expert_weights_norm, hp.expert_gating_func == "sigmoid",
                                        L.n_shared_merged or 0, hp.group_score_top2)
                base = self.expert_base if self.spec.expert_parallel else 0
                part = ops.moe_ffn(g, None, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, L.w_gate_sh, L.w_up_sh,
                                   L.w_down_sh, base)
                x = comm.reduce_scatter_rows(part, y)
        x_full = comm.all_gather_rows(x, final=True)
        xo = ops.select_rows(x_full, batch.out_rows) if batch.out_rows is not None else x_full[:T]
        xo, _ = ops.rmsnorm(xo, self.out_norm, hp.rms_eps)
        return ops.linear(xo, self.w_out, out_dtype=torch.float32)

    def _forward_idle(self) -> None:
        """A data-parallel rank without tokens still serves its experts to the other ranks: it joins every MoE
        layer's dispatch / combine with zero rows (the reference's llama_empty_run, src/llama-execute-decode.cpp:367-394)."""
        hp = self.hp
        x = torch.empty(0, hp.n_embd, dtype=self.dtype, device=self.device)
        ids = torch.empty(0, hp.n_expert_used, dtype=torch.int32, device=self.device)
        wts = torch.empty(0, hp.n_expert_used, dtype=torch.float32, device=self.device)
        for L in self.layers:
            if L.is_moe:
                self.ep.moe_ffn(x, None, ids, wts, L.w_gate_exps, L.w_up_exps, L.w_down_exps, None)
        return None

    @torch.no_grad()
    def forward(self, batch: Optional[ForwardBatch], kv_cache: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """kv_cache [n_layer, n_slots, r+dr].  Returns fp32 logits [len(out_rows), n_vocab].
        ``batch=None`` (data-parallel attention only): this rank has no tokens in this step."""
        hp = self.hp
        if self.comm is not None:
            self.comm.begin_step()
        if self.ep is not None:
            self.ep.begin_step()
        if batch is None:
            return self._forward_idle()
        sp_min = getattr(self.comm, "sp_min_tokens", 0) if self.comm is not None else 0
        if sp_min and self.spec.sharded and not self.spec.dp_attention and batch.tokens.shape[0] >= sp_min and batch.max_q_len > 1:
            return self._forward_sp(batch, kv_cache)
        x = ops.embed_gather(self.tok_embd, batch.tokens)
        nvtx = _trace.nvtx_enabled()
        by_dev = {self.device: batch}
        # single process, single device: a MoE block's combine can also produce the next block's attention norm
        fuse_norm = (ops.fused_combine_norm() and not self.spec.sharded and not self.split) or \
            (self.spec.sharded and not self.spec.dp_attention and getattr(self.comm, "fused_combine", False)
             and getattr(self.comm, "fused", False) and x.is_cuda and x.shape[0] <= self.comm.max_rows)
        h_next = None
        for il, L in enumerate(self.layers):
            if self.split:
                dev = self.layer_dev[il]
                if x.device != dev:
                    x = x.to(dev, non_blocking=True)          # the hop between two layer ranges
                    if dev.type == "cuda":
                        torch.cuda.set_device(dev)            # launches follow the current device's stream
                batch = by_dev.get(dev)
                if batch is None:
                    batch = by_dev[dev] = _batch_to(by_dev[self.device], dev)
            if nvtx:
                torch.cuda.nvtx.range_push(f"layer{il}")
            h = h_next if h_next is not None else ops.rmsnorm(x, L.attn_norm, hp.rms_eps)[0]
            h_next = None
            a = self._attention(L, h, batch, kv_cache[il])
            y = self._row_parallel(a, L.w_o, x)
            if fuse_norm and L.is_moe and il + 1 < len(self.layers):
                x, h_next = self._mlp(L, y, norm=(self.layers[il + 1].attn_norm, hp.rms_eps))
            else:
                x = self._mlp(L, y)
            if self.tensor_hook is not None:
                self.tensor_hook(f"blk.{il}.attn_out", a)
                self.tensor_hook(f"blk.{il}.ffn_inp", y)
                self.tensor_hook(f"blk.{il}.ffn_out", x)
            if nvtx:
                torch.cuda.nvtx.range_pop()
        xo = ops.select_rows(x, batch.out_rows) if batch.out_rows is not None else x
        xo, _ = ops.rmsnorm(xo, self.out_norm, hp.rms_eps)
        logits = ops.linear(xo, self.w_out, out_dtype=torch.float32)
        if self.tensor_hook is not None:
            self.tensor_hook("result_norm", xo)
            self.tensor_hook("result_output", logits)
        if self.split and self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        return logits
