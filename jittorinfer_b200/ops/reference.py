"""Plain-PyTorch implementations of every op the model graph uses.

These are (a) the CPU path (tests, host-only tools), (b) the fp32 numerics reference the CUDA
kernels are tested against, and (c) on a GPU, the torch/cuBLAS *baseline* the native kernels are
measured against (``JITTORINFER_OPS=torch``).  Semantics follow the reference graph
(src/llama-graph-deepseek2.cpp:113-405); each function names the reference op it stands for.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def embed_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """ggml get_rows on the token embedding (src/llama-graph-utils.cpp:7-40)."""
    return table[ids.long()]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(normed, summed): summed = x + residual (or x); normed = rmsnorm(summed) * w in fp32 statistics."""
    s = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    sf = s.float()
    n = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return n.to(x.dtype), s


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ w.T (+ residual); fp32 accumulate."""
    if x.dtype == torch.float32 or x.is_cuda:
        y = x @ w.T if out_dtype in (None, x.dtype) else (x.float() @ w.float().T)
    else:
        y = (x.float() @ w.float().T)
    if residual is not None:
        y = y.float() + residual.float()
    return y.to(out_dtype or x.dtype)


def gateup_silu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor) -> torch.Tensor:
    """silu(x wg^T) * (x wu^T) (src/llama-graph-ffn.cpp:4-126, LLM_FFN_SILU + LLM_FFN_PAR)."""
    g = linear(x, wg, out_dtype=torch.float32)
    u = linear(x, wu, out_dtype=torch.float32)
    return (F.silu(g) * u).to(x.dtype)


def yarn_table(n_pos: int, dr: int, freq_base: float, freq_scale: float, ext_factor: float, attn_factor: float,
               corr_lo: float, corr_hi: float, device="cpu") -> torch.Tensor:
    """[n_pos, dr/2, 2] fp32 (cos, sin) incl. magnitude factor — the GE path's RopeCache
    (ggml/src/ggml-cann/rope_cache.cpp:16-79) restated; formula ggml-cpu.c:10272-10305."""
    i = torch.arange(dr // 2, dtype=torch.float64)
    pos = torch.arange(n_pos, dtype=torch.float64)
    te = pos[:, None] * freq_base ** (-2.0 * i / dr)[None, :]
    ti = freq_scale * te
    if ext_factor != 0.0:
        ramp = 1.0 - torch.clamp((i - corr_lo) / max(0.001, corr_hi - corr_lo), 0.0, 1.0)
        mix = ramp * ext_factor
        theta = ti * (1.0 - mix) + te * mix
        m = attn_factor * (1.0 + 0.1 * math.log(1.0 / freq_scale))
    else:
        theta, m = ti, attn_factor
    return torch.stack([torch.cos(theta) * m, torch.sin(theta) * m], dim=-1).float().to(device)


def _rope(x: torch.Tensor, cs: torch.Tensor) -> torch.Tensor:
    # x [T, ..., dr]; cs [T, dr/2, 2]
    shp = x.shape
    xp = x.float().reshape(*shp[:-1], shp[-1] // 2, 2)
    c, s = cs[..., 0], cs[..., 1]
    while c.dim() < xp.dim() - 1:
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    x0, x1 = xp[..., 0], xp[..., 1]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).reshape(shp)


def mla_qkv_post(q: torch.Tensor, ckv: torch.Tensor, kv_norm_w: torch.Tensor, eps: float, rope_table: torch.Tensor,
                 positions: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                 q_out: torch.Tensor, n_head: int, dn: int, dr: int, r: int) -> torch.Tensor:
    """RMSNorm(c) + RoPE(k_pe) + latent-cache write + RoPE(q_pe)  (src/llama-graph-deepseek2.cpp:197-240).

    q [T, H*(dn+dr)], ckv [T, r+dr]; cache [n_slots, r+dr]; q_out [T, H, r+dr]: only the rope tail
    ``q_out[..., r:]`` is written here (the nope part is absorbed by :func:`q_absorb`).
    Rows with ``slot_mapping < 0`` are padding and are skipped.  Returns q_nope [T,H,dn] (a view).
    """
    T = q.shape[0]
    cs = rope_table[positions.long()]
    c = ckv[:, :r].float()
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * kv_norm_w.float()
    kpe = _rope(ckv[:, r:], cs)
    row = torch.cat([c, kpe], dim=-1).to(cache.dtype)
    valid = slot_mapping >= 0
    cache[slot_mapping[valid].long()] = row[valid]
    qv = q.view(T, n_head, dn + dr)
    q_out[..., r:] = _rope(qv[..., dn:], cs).to(q_out.dtype)
    return qv[..., :dn]


def q_absorb(q_nope: torch.Tensor, w_uk: torch.Tensor, q_out: torch.Tensor, r: int) -> None:
    """q_out[..., :r] = q_nope[T,H,dn] @ w_uk[H,r,dn]^T  (src/llama-graph-attn.cpp:269-275)."""
    q_out[..., :r] = torch.einsum("thd,hrd->thr", q_nope.float(), w_uk.float()).to(q_out.dtype)


def v_up(o_lat: torch.Tensor, w_uv: torch.Tensor) -> torch.Tensor:
    """o[T, H*dv] = o_lat[T,H,r] @ w_uv[H,dv,r]^T  (src/llama-graph-attn.cpp:316-317)."""
    o = torch.einsum("thr,hvr->thv", o_lat.float(), w_uv.float())
    return o.reshape(o.shape[0], -1).to(o_lat.dtype)


def mla_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                  q_start: torch.Tensor, scale: float, r: int, block_size: int) -> torch.Tensor:
    """Weight-absorbed MLA over the paged latent cache (src/llama-graph-attn.cpp:219-342).

    q [T,H,r+dr]; cache [n_blocks*block_size, r+dr]; sequence b owns query rows
    q_start[b]:q_start[b+1] (its *last* tokens) and kv length seq_lens[b].  Returns o_lat [T,H,r].
    """
    T, H, _ = q.shape
    out = torch.zeros(T, H, r, dtype=q.dtype, device=q.device)
    qs = q_start.tolist()
    sl = seq_lens.tolist()
    for b in range(len(sl)):
        q0, q1, S = qs[b], qs[b + 1], sl[b]
        if q1 <= q0 or S <= 0:
            continue
        nb = (S + block_size - 1) // block_size
        blocks = block_tables[b, :nb].long()
        idx = (blocks[:, None] * block_size + torch.arange(block_size, device=q.device)[None, :]).reshape(-1)[:S]
        lat = cache[idx].float()                                   # [S, r+dr]
        qq = q[q0:q1].float()                                      # [Tq,H,r+dr]
        s = torch.einsum("thk,sk->hts", qq, lat) * scale
        Tq = q1 - q0
        pos = S - Tq + torch.arange(Tq, device=q.device)
        vis = torch.arange(S, device=q.device)[None, :] <= pos[:, None]
        s = s.masked_fill(~vis[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("hts,sr->thr", p, lat[:, :r]).to(q.dtype)
    return out


def moe_gate(g: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], k: int, n_group: int,
             topk_group: int, scale: float, norm: bool, sigmoid: bool, n_shared: int = 0,
             group_top2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router matmul (fp32) + softmax/sigmoid + [group-limited] top-k + renorm/scale
    (src/llama-graph-ffn.cpp:145-197).  Returns ids [T,k] int32, weights [T,k] fp32."""
    logits = g.float() @ w_router.float().T
    probs = torch.sigmoid(logits) if sigmoid else torch.softmax(logits, dim=-1)
    sel = probs if bias is None else probs + bias.float()
    T, E = sel.shape
    if n_group > 1:
        grouped = sel.view(T, n_group, E // n_group)
        gs = grouped.topk(2, dim=-1).values.sum(-1) if group_top2 and E // n_group >= 2 else grouped.max(dim=-1).values
        order = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :topk_group]
        mask = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, order, True)
        sel = sel.masked_fill(~mask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    ids = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(probs, 1, ids)
    if norm:
        w = w / w.sum(-1, keepdim=True)
    ids, w = ids.int(), (w * scale).float()
    if n_shared:        # shared experts as always-selected experts E, E+1, ... with weight 1
        sh = torch.arange(E, E + n_shared, dtype=torch.int32, device=ids.device)[None].expand(T, n_shared)
        ids = torch.cat([ids, sh], dim=1)
        w = torch.cat([w, torch.ones(T, n_shared, dtype=w.dtype, device=w.device)], dim=1)
    return ids.contiguous(), w.contiguous()


def moe_experts(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor,
                wd: torch.Tensor, expert_base: int = 0) -> torch.Tensor:
    """sum_k w_k * down_e(silu(gate_e x) * up_e x) over the *local* experts
    [expert_base, expert_base + wg.shape[0]) (ggml_moe_fused with start/end expert,
    src/llama-graph-ffn.cpp:205-234).  Returns fp32 [T, d]."""
    T, d = x.shape
    E_local = wg.shape[0]
    out = torch.zeros(T, d, dtype=torch.float32, device=x.device)
    ids_l = ids.long() - expert_base
    for e in range(E_local):
        tok, slot = torch.nonzero(ids_l == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = gateup_silu(xe, wg[e], wu[e])
        y = linear(h, wd[e], out_dtype=torch.float32)
        out.index_add_(0, tok, y * wts[tok, slot][:, None])
    return out


def moe_ffn(x, residual, ids, wts, wg, wu, wd, wgs, wus, wds, expert_base=0):
    """residual + shared_experts(x) + routed experts (src/llama-graph-deepseek2.cpp:343-362)."""
    out = moe_experts(x, ids, wts, wg, wu, wd, expert_base)
    if wgs is not None:
        out = out + linear(gateup_silu(x, wgs, wus), wds, out_dtype=torch.float32)
    if residual is not None:
        out = out + residual.float()
    return out.to(x.dtype)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return torch.argmax(logits.float(), dim=-1).int()


def topk_logits(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Device "presample" (src/llama-execute-decode.cpp:132-154): top-k values fp32 + ids int32, sorted."""
    v, i = torch.topk(logits.float(), k, dim=-1, sorted=True)
    return v, i.int()


def sample_topk(vals: torch.Tensor, ids: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """One token id per row from its top-k candidates, the device form of the chain top_k -> top_p -> min_p -> temperature
    -> dist (common/sampling_local.cpp:153-209).  ``vals`` / ``ids`` [n, k] sorted by value, descending; ``params`` [n, 5]
    fp32 = temperature (<= 0: best candidate), top_k (<= 0: all), top_p (>= 1: off), min_p (<= 0: off), u in [0, 1).
    Sorted candidates make every truncation a prefix: rank < top_k; probability mass before the candidate < top_p (softmax
    of the untempered logits of the top-k set); logit >= best + ln(min_p)."""
    v = vals.float()
    n, k = v.shape
    pr = params.float()
    temp, top_k, top_p, min_p, u = (pr[:, i:i + 1] for i in range(5))
    rank = torch.arange(k, device=v.device)[None]
    keep = (top_k <= 0) | (rank < top_k)
    m = v[:, :1]
    e = torch.exp(v - m) * keep
    before = (torch.cumsum(e, -1) - e) / e.sum(-1, keepdim=True)
    keep = keep & ((top_p >= 1.0) | (before < top_p))
    keep = keep & ((min_p <= 0) | (v >= m + torch.log(min_p.clamp_min(1e-30))))
    keep[:, 0] = True
    keep = torch.cumprod(keep.int(), -1).bool()                       # a prefix, as the sequential form breaks at the first miss
    w = torch.exp((v - m) / temp.clamp_min(1e-6)) * keep
    cdf = torch.cumsum(w, -1)
    pick = (cdf <= u * cdf[:, -1:]).sum(-1)
    last = keep.sum(-1) - 1
    pick = torch.minimum(pick, last)
    pick = torch.where(temp[:, 0] <= 0, torch.zeros_like(pick), pick)
    return ids.gather(1, pick[:, None].long())[:, 0].int()


def kv_block_copy(cache: torch.Tensor, src_blocks: torch.Tensor, dst_blocks: torch.Tensor, block_size: int) -> None:
    """Defrag move list (src/llama-graph-defrag.cpp:23-85) on paged blocks. cache [L, n_slots, row]."""
    L = cache.shape[0]
    c = cache.view(L, -1, block_size, cache.shape[-1])
    c[:, dst_blocks.long()] = c[:, src_blocks.long()]
