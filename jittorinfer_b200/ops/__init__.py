"""Op front-end used by the model graph.

CUDA tensors go to the hand-written sm_100a kernels (``ops.native``, loaded from the in-tree
``libjib200_kernels.so``); if that library is missing on a GPU machine the import fails loudly —
there is no silent fallback.  CPU tensors (tests, host tools) use ``ops.reference``.
``JITTORINFER_OPS=torch`` selects the PyTorch/cuBLAS implementation on the GPU as well: that is
the measured baseline, never the default.
"""
from __future__ import annotations

import os

import torch

from . import reference as ref

_FORCE_TORCH = os.environ.get("JITTORINFER_OPS", "").lower() == "torch"
_native = None


def nat():
    """The ctypes binding module; raises if the CUDA library is not built."""
    global _native
    if _native is None:
        from . import native as _n
        _n.load()
        _native = _n
    return _native


def use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_TORCH


def set_force_torch(flag: bool) -> None:
    global _FORCE_TORCH
    _FORCE_TORCH = bool(flag)


def force_torch() -> bool:
    return _FORCE_TORCH


def embed_gather(table, ids):
    return nat().embed_gather(table, ids) if use_native(table) else ref.embed_gather(table, ids)


def select_rows(x, rows):
    """x[rows] (the reference's inp_out_ids row selection, src/llama-graph-deepseek2.cpp:302-308)."""
    if use_native(x) and x.dtype == torch.bfloat16:
        return nat().gather_rows(x, rows)
    return x[rows.long()].contiguous()


def rmsnorm(x, w, eps, residual=None):
    return nat().rmsnorm(x, w, eps, residual) if use_native(x) else ref.rmsnorm(x, w, eps, residual)


def linear(x, w, residual=None, out_dtype=None):
    if use_native(x) and x.dtype == torch.bfloat16:
        return nat().linear(x, w, residual, out_dtype)
    return ref.linear(x, w, residual, out_dtype)


def gateup_silu(x, wg, wu):
    if use_native(x) and x.dtype == torch.bfloat16:
        return nat().gateup_silu(x, wg, wu)
    return ref.gateup_silu(x, wg, wu)


def mla_qkv_post(q, ckv, kv_norm_w, eps, rope_table, positions, slot_mapping, cache, q_out, n_head, dn, dr, r):
    f = nat().mla_qkv_post if use_native(q) else ref.mla_qkv_post
    return f(q, ckv, kv_norm_w, eps, rope_table, positions, slot_mapping, cache, q_out, n_head, dn, dr, r)


def q_absorb(q_nope, w_uk, q_out, r):
    return (nat().q_absorb if use_native(q_nope) else ref.q_absorb)(q_nope, w_uk, q_out, r)


def v_up(o_lat, w_uv):
    return (nat().v_up if use_native(o_lat) else ref.v_up)(o_lat, w_uv)


def mla_attention(q, cache, block_tables, seq_lens, q_start, scale, r, block_size, max_q_len=None, meta=None):
    if use_native(q):
        return nat().mla_attention(q, cache, block_tables, seq_lens, q_start, scale, r, block_size, max_q_len, meta)
    return ref.mla_attention(q, cache, block_tables, seq_lens, q_start, scale, r, block_size)


def moe_gate(g, w_router, bias, k, n_group, topk_group, scale, norm, sigmoid, n_shared=0, group_top2=False, route=None, pre_norm=None):
    """``route=(expert_base, E_local)`` tells the CUDA path which local expert sort follows (see ``native.moe_gate``).
    ``pre_norm=(weight, eps)``: ``g`` is the un-normalised block input; returns (ids, wts, rmsnorm(g) * weight) -- on the CUDA
    path the router launch of a decode batch normalises the rows itself."""
    if use_native(g):
        return nat().moe_gate(g, w_router, bias, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2, route, pre_norm)
    if pre_norm is not None:
        g, _ = ref.rmsnorm(g, pre_norm[0], pre_norm[1])
        return ref.moe_gate(g, w_router, bias, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2) + (g,)
    return ref.moe_gate(g, w_router, bias, k, n_group, topk_group, scale, norm, sigmoid, n_shared, group_top2)


def moe_experts(x, ids, wts, wg, wu, wd, expert_base=0):
    if use_native(x) and x.dtype == torch.bfloat16:
        return nat().moe_experts(x, ids, wts, wg, wu, wd, expert_base)
    return ref.moe_experts(x, ids, wts, wg, wu, wd, expert_base)


def moe_ffn(x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base=0, n_expert=None, norm=None):
    """``n_expert``: size of the router's expert set (lets the CUDA path estimate how many local experts a batch hits).
    ``norm=(weight, eps)``: returns (out, rmsnorm(out) * weight) -- the CUDA path computes both in the combine launch."""
    if use_native(x) and x.dtype == torch.bfloat16:
        return nat().moe_ffn(x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base, n_expert, norm)
    out = ref.moe_ffn(x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base)
    return (out, ref.rmsnorm(out, norm[0], norm[1])[0]) if norm is not None else out


def fused_combine_norm() -> bool:
    """Whether the model should ask ``moe_ffn`` for the next block's norm as well (one launch on the CUDA path;
    JIB_FUSED_COMBINE_NORM=0 keeps the two launches for A/B measurements)."""
    return os.environ.get("JIB_FUSED_COMBINE_NORM", "1") == "1"


def argmax(logits):
    return nat().argmax(logits) if use_native(logits) else ref.argmax(logits)


def topk_logits(logits, k):
    return nat().topk_logits(logits, k) if use_native(logits) else ref.topk_logits(logits, k)


def sample_topk(vals, ids, params):
    """One id per row from sorted top-k candidates: top-k / top-p / min-p / temperature and one uniform per row."""
    return nat().sample_topk(vals, ids, params) if use_native(vals) else ref.sample_topk(vals, ids, params)


def kv_block_copy(cache, src_blocks, dst_blocks, block_size):
    f = nat().kv_block_copy if use_native(cache) else ref.kv_block_copy
    return f(cache, src_blocks, dst_blocks, block_size)
