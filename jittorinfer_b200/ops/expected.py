"""Expected memory time of every launch of one decode step: the figures to hold a measurement against.

Decode at small batch is a weight stream: each launch's lower bound is the bytes it must read (weights it touches, cache
rows, activations) divided by the copy bandwidth of the GPU.  This tool lists the launches of one MoE layer in the order
the model issues them (``models/deepseek2.py``), their algorithmic bytes and the time those bytes take at the given
bandwidth, then the whole step -- so that a measured step, or a per-op breakdown from ``ops/profile.py``, can be read as
"x times the memory time" launch by launch.  Routed-expert traffic uses the expected number of distinct experts hit under
uniform routing, ``E_local * (1 - (1 - k/E)^T)``.

    python -m jittorinfer_b200.ops.expected --model lite --tokens 8 --cached 1100
    python -m jittorinfer_b200.ops.expected --model v2 --world 8 --tokens 8 --cached 1100 --measured-ms 15.27 --launches 1199
    python -m jittorinfer_b200.ops.expected --model lite --prefill 2048 --measured-ms 55          # a prefill chunk: FLOPs and bytes

The bandwidth defaults to ``hbm_gbs`` of a ``MEASURED_PEAKS.json`` next to the package if there is one, else 6.65 TB/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Tuple

from ..models.hparams import DeepSeek2HParams, preset


def default_bandwidth() -> float:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]) * 1e9
    except (OSError, KeyError, ValueError):
        return 6.65e12


def layer_launches(hp: DeepSeek2HParams, T: int, S: int, world: int = 1) -> List[Tuple[str, float, str]]:
    """(launch, bytes, note) of one MoE layer for ``T`` sequences with ``S`` cached tokens each, per rank of ``world``."""
    d, H = hp.n_embd, hp.n_head // world
    dn, dr, dv, r = hp.qk_nope_head_dim, hp.qk_rope_head_dim, hp.v_head_dim, hp.kv_lora_rank
    E, k, nff, sh = hp.n_expert, hp.n_expert_used, hp.n_ff_exp, hp.n_expert_shared
    out: List[Tuple[str, float, str]] = []

    def add(kern, byts, note=""):
        out.append((kern, float(byts), note))
    add("rmsnorm (attn_norm)", T * d * 2 * 2)
    if hp.q_lora_rank:
        add("GEMM q_a + kv_a", (hp.q_lora_rank + r + dr) * d * 2)
        add("rmsnorm (q_a_norm)", T * hp.q_lora_rank * 4)
        add("GEMM q_b", H * (dn + dr) * hp.q_lora_rank * 2)
    else:
        add("GEMM q + kv_a", (H * (dn + dr) + r + dr) * d * 2)
    add("mla_qkv_post (kv norm, RoPE, cache write)", T * (H * (dn + dr) + r + dr) * 2 * 2)
    add("GEMM q_absorb (batched per head)", H * dn * r * 2)
    add("flash MLA (split-KV)", T * S * (r + dr) * 2, f"{T} sequences x {S} cached tokens")
    add("mla_combine", T * 8 * H * r * 4, "~8 splits of fp32 partials")
    add("GEMM v_up (batched per head)", H * r * dv * 2)
    add("GEMM o_proj (+ residual" + (", + all-reduce" if world > 1 else "") + ")", d * H * dv * 2)
    add("rmsnorm (ffn_norm)", T * d * 2 * 2)
    add("router logits (fp32)", E * d * 4)
    add("gate (top-k)", T * E * 4)
    add("expert sort", T * k * 4 * 3)
    add("gather rows", T * k * d * 2 * 2)
    e_local = E // world
    hit = e_local * (1 - (1 - k / E) ** T)
    if world == 1:
        add("grouped GEMM gate|up (+ shared experts merged)", (hit + sh) * 2 * nff * d * 2, f"{hit:.1f} of {e_local} routed experts hit")
        add("grouped GEMM down", (hit + sh) * nff * d * 2)
        add("combine (+ residual)", T * (k + sh) * d * 2)
    else:
        add("grouped GEMM gate|up", hit * 2 * nff * d * 2, f"{hit:.1f} of {e_local} local experts hit")
        add("grouped GEMM down", hit * nff * d * 2)
        add("GEMM shared gate|up", 2 * sh * nff // world * d * 2)
        add("GEMM shared down", sh * nff // world * d * 2)
        add("combine", T * k * d * 2)
        add("all-reduce (+ residual)", T * d * 4 * (world - 1), "bytes pushed over NVLink per rank")
    return out


def step_memory_bytes(hp: DeepSeek2HParams, T: int, S: int, world: int = 1) -> float:
    """Bytes one rank must read in one decode step of ``T`` sequences with ``S`` cached tokens each: every layer's launches
    (dense leading layers stream their whole FFN instead of the experts hit) plus the output head.  Divided by the copy
    bandwidth this is the memory-bound time a measured step is held against."""
    rows = layer_launches(hp, T, S, world)
    moe = sum(b for _, b, _ in rows)
    attn = sum(b for k, b, _ in rows[: next(i for i, r in enumerate(rows) if r[0].startswith("rmsnorm (ffn_norm)")) + 1])
    dense = attn + 3 * hp.n_ff * hp.n_embd * 2 / world
    head = hp.n_vocab * hp.n_embd * 2
    n_dense = hp.n_layer_dense_lead if hp.n_layer > hp.n_layer_dense_lead else 0
    return n_dense * dense + (hp.n_layer - n_dense) * moe + head


def prefill_launches(hp: DeepSeek2HParams, T: int, world: int = 1) -> List[Tuple[str, float, float, str]]:
    """(launch, FLOPs, bytes, note) of one MoE layer for a prefill chunk of ``T`` tokens of one sequence (causal), per rank."""
    d, H = hp.n_embd, hp.n_head // world
    dn, dr, dv, r = hp.qk_nope_head_dim, hp.qk_rope_head_dim, hp.v_head_dim, hp.kv_lora_rank
    E, k, nff, sh = hp.n_expert, hp.n_expert_used, hp.n_ff_exp, hp.n_expert_shared
    out: List[Tuple[str, float, float, str]] = []

    def gemm(kern, n, kk, rows=T, note="", weights=None):
        out.append((kern, 2.0 * rows * n * kk, float((weights if weights is not None else n * kk) * 2 + rows * (n + kk) * 2), note))

    def elem(kern, byts, note=""):
        out.append((kern, 0.0, float(byts), note))
    elem("rmsnorm (attn_norm)", T * d * 2 * 2)
    if hp.q_lora_rank:
        gemm("GEMM q_a + kv_a", hp.q_lora_rank + r + dr, d)
        elem("rmsnorm (q_a_norm)", T * hp.q_lora_rank * 4)
        gemm("GEMM q_b", H * (dn + dr), hp.q_lora_rank)
    else:
        gemm("GEMM q + kv_a", H * (dn + dr) + r + dr, d)
    elem("mla_qkv_post (kv norm, RoPE, cache write)", T * (H * (dn + dr) + r + dr) * 2 * 2)
    if (dn, dr, dv, r) == (128, 64, 128, 512) and T >= 64:
        # prompt chunks at the DeepSeek head sizes run the per-head form: K / V expanded from the latent rows by one GEMM
        elem("kv gather (latent rows of the chunk's sequences)", T * (r + dr) * 2 * 2)
        gemm("GEMM K/V expansion (k_nope | v per head)", H * (dn + dv), r)
        out.append(("prompt attention (per head, causal)", 2.0 * H * (T * (T + 1) / 2) * ((dn + dr) + dv),
                    float(T * H * (dn + dr) * 2 + T * H * (dn + dv) * 2 + T * dr * 2 + T * H * dv * 2), "scores over 192 dims, values over 128"))
    else:
        gemm("GEMM q_absorb (batched per head)", H * r, dn, note="per head 128 -> 512", weights=H * dn * r)
        out.append(("flash MLA (absorbed, causal)", 2.0 * H * (T * T / 2) * ((r + dr) + r), float(T * (r + dr) * 2 + T * H * (2 * r + dr) * 2),
                    "scores over 576 dims, values over 512"))
        gemm("GEMM v_up (batched per head)", H * dv, r, note="per head 512 -> 128", weights=H * r * dv)
    gemm("GEMM o_proj (+ residual" + (", + all-reduce" if world > 1 else "") + ")", d, H * dv)
    elem("rmsnorm (ffn_norm)", T * d * 2 * 2)
    out.append(("router logits (fp32)", 2.0 * T * E * d, float(E * d * 4 + T * d * 2), ""))
    elem("gate (top-k)", T * E * 4)
    elem("expert sort", T * k * 4 * 4)
    elem("gather rows", T * k * d * 2 * 2)
    e_local = E // world
    pairs = T * k / world if world > 1 else T * (k + sh)          # rows that reach this rank's experts
    n_exp = e_local + (sh if world == 1 else 0)
    gemm("grouped GEMM gate|up", 2 * nff, d, rows=pairs, weights=n_exp * 2 * nff * d, note=f"{pairs / n_exp:.0f} rows per expert")
    gemm("grouped GEMM down", d, nff, rows=pairs, weights=n_exp * nff * d)
    if world > 1:
        gemm("GEMM shared gate|up", 2 * sh * nff // world, d)
        gemm("GEMM shared down", d, sh * nff // world)
    elem("combine (+ residual)", T * (k + 2) * d * 2)
    if world > 1:
        elem("all-reduce (two-shot)", T * d * (4 + 2) * (world - 1) / world, "bytes over NVLink per rank")
    return out


def report_prefill(hp: DeepSeek2HParams, T: int, world: int, bandwidth: float, tflops: float, measured_ms: float = 0.0) -> str:
    rows = prefill_launches(hp, T, world)
    lines = [f"| launch | GFLOP | MB | bound, us (max of {tflops:.0f} TFLOP/s and {bandwidth / 1e12:.2f} TB/s) | note |", "|---|---|---|---|---|"]
    total = 0.0
    for kern, fl, b, note in rows:
        t = max(fl / (tflops * 1e12), b / bandwidth) * 1e6
        total += t
        lines.append(f"| {kern} | {fl / 1e9:.1f} | {b / 1e6:.1f} | {t:.1f} | {note} |")
    lines.append(f"| **one MoE layer, {T} tokens** | {sum(r[1] for r in rows) / 1e9:.0f} | {sum(r[2] for r in rows) / 1e6:.0f} | **{total:.0f}** | {len(rows)} launches |")
    n_moe = hp.n_layer - hp.n_layer_dense_lead
    tail = f"\n{hp.n_layer} layers x ~{total:.0f} us = {hp.n_layer * total / 1e3:.1f} ms per {T}-token chunk at the bound"
    if measured_ms > 0:
        tail += f"; measured ~{measured_ms} ms ({hp.n_layer * total / 1e3 / measured_ms:.2f} of the bound)"
    return "\n".join(lines) + tail + "."


def report(hp: DeepSeek2HParams, T: int, S: int, world: int, bandwidth: float, measured_ms: float = 0.0, launches: int = 0) -> str:
    rows = layer_launches(hp, T, S, world)
    us = [b / bandwidth * 1e6 for _, b, _ in rows]
    lines = [f"| launch | bytes | memory time, us at {bandwidth / 1e12:.2f} TB/s | note |", "|---|---|---|---|"]
    for (kern, b, note), t in zip(rows, us):
        lines.append(f"| {kern} | {b / 1e6:.2f} MB | {t:.2f} | {note} |")
    lines.append(f"| **one MoE layer** | {sum(b for _, b, _ in rows) / 1e6:.1f} MB | **{sum(us):.1f}** | {len(rows)} launches |")
    n_moe = hp.n_layer - hp.n_layer_dense_lead
    head = hp.n_vocab * hp.n_embd * 2 / bandwidth * 1e6
    total = n_moe * sum(us) + head
    tail = f"\n{n_moe} MoE layers x {sum(us):.1f} us + lm_head {head:.0f} us = {total / 1e3:.2f} ms of memory time per step"
    if measured_ms > 0 and launches > 0:
        tail += (f"; measured {measured_ms} ms with {launches} launches = {measured_ms * 1e3 / launches:.1f} us per launch against "
                 f"{total / launches:.1f} us of memory time per launch ({total / 1e3 / measured_ms:.2f} of the bound)")
    return "\n".join(lines) + tail + "."


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="lite")
    ap.add_argument("--tokens", type=int, default=8, help="sequences in the decode step")
    ap.add_argument("--cached", type=int, default=1100, help="cached tokens per sequence")
    ap.add_argument("--world", type=int, default=1, help="tensor/expert-parallel ranks")
    ap.add_argument("--bandwidth-gbs", type=float, default=0.0, help="copy bandwidth in GB/s (default: measured peaks file, else 6650)")
    ap.add_argument("--measured-ms", type=float, default=0.0)
    ap.add_argument("--launches", type=int, default=0)
    ap.add_argument("--prefill", type=int, default=0, help="instead of a decode step: one prefill chunk of this many tokens")
    ap.add_argument("--tflops", type=float, default=1360.0, help="sustained bf16 GEMM rate for the prefill bound")
    a = ap.parse_args(argv)
    bw = a.bandwidth_gbs * 1e9 if a.bandwidth_gbs > 0 else default_bandwidth()
    if a.prefill > 0:
        print(report_prefill(preset(a.model), a.prefill, a.world, bw, a.tflops, a.measured_ms))
    else:
        print(report(preset(a.model), a.tokens, a.cached, a.world, bw, a.measured_ms, a.launches))
    return 0


if __name__ == "__main__":
    sys.exit(main())
