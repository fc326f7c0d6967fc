"""fp32 PyTorch restatement of the reference's DeepSeek-V2 forward pass — the numerical oracle.

Every step follows the graph the reference builds in ``llm_deepseek2_context::build_deepseek2``
(src/llama-graph-deepseek2.cpp:113-405), ``llm_attn_mla`` / ``llm_build_kv``
(src/llama-graph-attn.cpp:185-342) and ``llm_build_ffn`` / ``llm_build_moe_ffn``
(src/llama-graph-ffn.cpp:4-287); RoPE follows ggml's YaRN formula (ggml/src/ggml-cpu/ggml-cpu.c:
10272-10305).  Both attention forms are implemented (weight-absorbed MLA over the latent cache and
the naive per-head form); they are algebraically identical and the tests assert that they agree.
Group-limited routing (absent from the reference, src/llama-graph-ffn.cpp:174-177) follows the
DeepSeek-V2 model definition and is enabled only when ``n_group > 1``.

Nothing here is fast; it is written to be obviously correct.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .hparams import DeepSeek2HParams


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def yarn_cos_sin(hp: DeepSeek2HParams, pos: torch.Tensor):
    """cos/sin tables [T, dr/2] (already multiplied by the magnitude factor)."""
    dr = hp.qk_rope_head_dim
    i = torch.arange(dr // 2, dtype=torch.float64, device=pos.device)
    theta_extrap = pos.double()[:, None] * hp.rope_freq_base ** (-2.0 * i / dr)[None, :]
    s = hp.freq_scale
    theta_interp = s * theta_extrap
    ext = hp.ext_factor
    attn = hp.rope_attn
    if ext != 0.0:
        lo, hi = hp.yarn_corr_dims()
        ramp = 1.0 - torch.clamp((i - lo) / max(0.001, hi - lo), 0.0, 1.0)
        mix = ramp * ext
        theta = theta_interp * (1.0 - mix) + theta_extrap * mix
        m = attn * (1.0 + 0.1 * math.log(1.0 / s))
    else:
        theta = theta_interp
        m = attn
    return (torch.cos(theta) * m).float(), (torch.sin(theta) * m).float()


def rope_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs (x[2i], x[2i+1]).  x: [T, ..., dr]; cos/sin: [T, dr/2]."""
    shp = x.shape
    xp = x.float().reshape(*shp[:-1], shp[-1] // 2, 2)
    while cos.dim() < xp.dim() - 1:
        cos = cos.unsqueeze(1)
        sin = sin.unsqueeze(1)
    x0, x1 = xp[..., 0], xp[..., 1]
    out = torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)
    return out.reshape(shp)


def gate_topk(hp: DeepSeek2HParams, logits: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """logits [T,E] fp32 -> (ids [T,k] int64, weights [T,k] fp32)."""
    if hp.expert_gating_func == "sigmoid":
        probs = torch.sigmoid(logits.float())
    else:
        probs = torch.softmax(logits.float(), dim=-1)
    sel = probs if bias is None else probs + bias.float()
    if hp.n_group > 1:
        T, E = sel.shape
        g = sel.view(T, hp.n_group, E // hp.n_group)
        gscore = g.topk(2, dim=-1).values.sum(-1) if hp.group_score_top2 and g.shape[-1] >= 2 else g.max(dim=-1).values
        keep = torch.topk(gscore, hp.topk_group, dim=-1, sorted=False).indices
        mask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, keep, True)
        sel = sel.masked_fill(~mask[:, :, None].expand_as(g).reshape(T, E), float("-inf"))
    # stable descending order: ties resolved towards the lower expert id
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices
    ids = order[:, : hp.n_expert_used]
    w = torch.gather(probs, 1, ids)
    if hp.expert_weights_norm:
        w = w / w.sum(-1, keepdim=True)
    w = w * hp.expert_weights_scale
    return ids, w


def ffn(x, wg, wu, wd):
    return (torch.nn.functional.silu(x @ wg.float().T) * (x @ wu.float().T)) @ wd.float().T


class OracleModel:
    """Holds fp32 weights keyed by GGUF tensor names and a contiguous per-sequence cache."""

    def __init__(self, hp: DeepSeek2HParams, weights: Dict[str, torch.Tensor], absorbed: bool = True):
        self.hp = hp
        self.w = {k: v.float() for k, v in weights.items()}
        self.absorbed = absorbed
        self.reset()

    def reset(self):
        L = self.hp.n_layer
        self.lat: List[Optional[torch.Tensor]] = [None] * L     # [S, r+dr]
        self.k: List[Optional[torch.Tensor]] = [None] * L       # naive: [S, H, dk]
        self.v: List[Optional[torch.Tensor]] = [None] * L       # naive: [S, H, dv]
        self.n_past = 0

    # ---------------------------------------------------------------------------------------
    def _attn(self, il: int, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        hp, w = self.hp, self.w
        T = h.shape[0]
        H, dn, dr, dv, r = hp.n_head, hp.qk_nope_head_dim, hp.qk_rope_head_dim, hp.v_head_dim, hp.kv_lora_rank
        p = f"blk.{il}."
        if hp.is_lite:
            q = h @ w[p + "attn_q.weight"].T
        else:
            qa = rmsnorm(h @ w[p + "attn_q_a.weight"].T, w[p + "attn_q_a_norm.weight"], hp.rms_eps)
            q = qa @ w[p + "attn_q_b.weight"].T
        q = q.view(T, H, dn + dr)
        q_nope, q_pe = q[..., :dn], q[..., dn:]
        ckv = h @ w[p + "attn_kv_a_mqa.weight"].T
        c = rmsnorm(ckv[:, :r], w[p + "attn_kv_a_norm.weight"], hp.rms_eps)
        k_pe = ckv[:, r:]
        cos, sin = yarn_cos_sin(hp, pos)
        q_pe = rope_pairs(q_pe, cos, sin)
        k_pe = rope_pairs(k_pe, cos, sin)
        wkv_b = w[p + "attn_kv_b.weight"].view(H, dn + dv, r)
        n_past = self.n_past
        S = n_past + T
        # causal mask over [T, S]
        j = torch.arange(S)[None, :]
        vis = j <= (n_past + torch.arange(T))[:, None]
        bias = torch.zeros(T, S).masked_fill(~vis, float("-inf"))
        if self.absorbed:
            row = torch.cat([c, k_pe], dim=-1)
            self.lat[il] = row if self.lat[il] is None else torch.cat([self.lat[il][:n_past], row], 0)
            lat = self.lat[il]
            w_uk = wkv_b[:, :dn, :]                       # [H, dn, r]
            w_uv = wkv_b[:, dn:, :]                       # [H, dv, r]
            q_abs = torch.einsum("thd,hdr->thr", q_nope, w_uk)
            qq = torch.cat([q_abs, q_pe], dim=-1)         # [T,H,r+dr]
            s = torch.einsum("thk,sk->hts", qq, lat) * hp.kq_scale + bias[None]
            pr = torch.softmax(s, dim=-1)
            o_lat = torch.einsum("hts,sr->thr", pr, lat[:, :r])
            o = torch.einsum("thr,hvr->thv", o_lat, w_uv)
        else:
            kv = (c @ wkv_b.reshape(H * (dn + dv), r).T).view(T, H, dn + dv)
            k = torch.cat([kv[..., :dn], k_pe[:, None, :].expand(T, H, dr)], dim=-1)
            v = kv[..., dn:]
            self.k[il] = k if self.k[il] is None else torch.cat([self.k[il][:n_past], k], 0)
            self.v[il] = v if self.v[il] is None else torch.cat([self.v[il][:n_past], v], 0)
            qq = torch.cat([q_nope, q_pe], dim=-1)
            s = torch.einsum("thk,shk->hts", qq, self.k[il]) * hp.kq_scale + bias[None]
            pr = torch.softmax(s, dim=-1)
            o = torch.einsum("hts,shv->thv", pr, self.v[il])
        return o.reshape(T, H * dv) @ w[p + "attn_output.weight"].T

    def _mlp(self, il: int, g: torch.Tensor) -> torch.Tensor:
        hp, w = self.hp, self.w
        p = f"blk.{il}."
        if il < hp.n_layer_dense_lead:
            return ffn(g, w[p + "ffn_gate.weight"], w[p + "ffn_up.weight"], w[p + "ffn_down.weight"])
        logits = g @ w[p + "ffn_gate_inp.weight"].T
        ids, wt = gate_topk(hp, logits, w.get(p + "exp_probs_b.bias"))
        out = torch.zeros_like(g)
        wg, wu, wd = w[p + "ffn_gate_exps.weight"], w[p + "ffn_up_exps.weight"], w[p + "ffn_down_exps.weight"]
        for t in range(g.shape[0]):
            for kk in range(hp.n_expert_used):
                e = int(ids[t, kk])
                out[t] += wt[t, kk] * ffn(g[t:t + 1], wg[e], wu[e], wd[e])[0]
        if hp.n_expert_shared:
            out = out + ffn(g, w[p + "ffn_gate_shexp.weight"], w[p + "ffn_up_shexp.weight"], w[p + "ffn_down_shexp.weight"])
        return out

    def forward(self, tokens: torch.Tensor, n_past: Optional[int] = None) -> torch.Tensor:
        """tokens [T] appended at positions n_past..n_past+T-1 -> logits [T, n_vocab] fp32."""
        hp, w = self.hp, self.w
        if n_past is not None:
            self.n_past = n_past
        T = tokens.shape[0]
        pos = torch.arange(self.n_past, self.n_past + T)
        x = w["token_embd.weight"][tokens.long()]
        for il in range(hp.n_layer):
            p = f"blk.{il}."
            h = rmsnorm(x, w[p + "attn_norm.weight"], hp.rms_eps)
            y = x + self._attn(il, h, pos)
            g = rmsnorm(y, w[p + "ffn_norm.weight"], hp.rms_eps)
            x = y + self._mlp(il, g)
        self.n_past += T
        xo = rmsnorm(x, w["output_norm.weight"], hp.rms_eps)
        return xo @ w["output.weight"].T

    @torch.no_grad()
    def generate(self, prompt: List[int], n_new: int) -> List[int]:
        self.reset()
        logits = self.forward(torch.tensor(prompt))
        out = []
        for _ in range(n_new):
            nxt = int(torch.argmax(logits[-1]))
            out.append(nxt)
            logits = self.forward(torch.tensor([nxt]))
        return out
