"""Kernel micro-benchmarks with roofline fractions.

    python -m jittorinfer_b200.ops.microbench gemm --T 8 --N 32768 --K 2048
    python -m jittorinfer_b200.ops.microbench gateup --T 8 --N 16384 --K 2048
    python -m jittorinfer_b200.ops.microbench moe --T 8 --E 64 --k 6 --F 1408 --d 2048
    python -m jittorinfer_b200.ops.microbench attn --B 8 --S 1280
    python -m jittorinfer_b200.ops.microbench prefill_gemm --T 4096 --N 4096 --K 4096
    python -m jittorinfer_b200.ops.microbench prefill_attn --T 2048 --H 16

Each case is timed with CUDA events on the launching stream after warm-up (synchronise on both
sides); operands are larger than the 126 MB L2 or rotated over several buffers so that every
iteration streams from HBM.  Fractions are of the measured peaks in MEASURED_PEAKS.json
(fallback 6.65 TB/s, 1.59 PFLOP/s).  `--iters 1 --warmup 0` gives a run small enough for `ncu`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def report(name, ms, nbytes, flops, extra=None):
    hbm, tf, how = peaks()
    gbs = nbytes / ms / 1e6
    tfl = flops / ms / 1e9
    out = {"case": name, "ms": round(ms, 4), "GB/s": round(gbs, 1), "TFLOP/s": round(tfl, 1),
           f"frac_hbm_of_{how}": round(gbs / hbm, 3), f"frac_bf16_of_{how}": round(tfl / tf, 3)}
    if extra:
        out.update(extra)
    print(json.dumps(out))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gateup", "moe", "attn", "prefill_attn", "prefill_gemm", "route", "combine_norm", "permute", "sample"])
    ap.add_argument("--T", type=int, default=8)
    ap.add_argument("--N", type=int, default=32768)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--E", type=int, default=64)
    ap.add_argument("--k", type=int, default=6)
    ap.add_argument("--F", type=int, default=1408)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--S", type=int, default=1280)
    ap.add_argument("--H", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--torch", action="store_true", help="time the PyTorch/cuBLAS op instead (baseline)")
    a = ap.parse_args(argv)
    from . import native as nat
    nat.load()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).bfloat16()

    if a.case in ("gemm", "prefill_gemm"):
        n_buf = max(1, int(2.6e8 // (a.N * a.K * 2)) + 1)        # rotate weights so that each pass misses L2
        ws = [rnd(a.N, a.K, scale=0.05) for _ in range(n_buf)]
        x = rnd(a.T, a.K)
        i = [0]

        def fn():
            w = ws[i[0] % n_buf]
            i[0] += 1
            return (x @ w.T) if a.torch else nat.gemm(x, w, splits=a.splits)

        ms = timeit(fn, a.iters, a.warmup)
        report(f"{a.case} T={a.T} N={a.N} K={a.K}" + (" [torch]" if a.torch else ""), ms,
               a.N * a.K * 2 + a.T * (a.N + a.K) * 2, 2.0 * a.T * a.N * a.K)
    elif a.case == "gateup":
        n_buf = max(1, int(2.6e8 // (2 * a.N * a.K * 2)) + 1)
        wg = [rnd(a.N, a.K, scale=0.05) for _ in range(n_buf)]
        wu = [rnd(a.N, a.K, scale=0.05) for _ in range(n_buf)]
        x = rnd(a.T, a.K)
        i = [0]

        def fn():
            j = i[0] % n_buf
            i[0] += 1
            if a.torch:
                return torch.nn.functional.silu(x @ wg[j].T) * (x @ wu[j].T)
            return nat.gemm(x, wg[j], wu[j], splits=a.splits)

        ms = timeit(fn, a.iters, a.warmup)
        report(f"gateup T={a.T} N={a.N} K={a.K}" + (" [torch]" if a.torch else ""), ms, 2 * a.N * a.K * 2, 4.0 * a.T * a.N * a.K)
    elif a.case == "moe":
        E, k, F, d, T = a.E, a.k, a.F, a.d, a.T
        wg, wu, wd = rnd(E, F, d, scale=0.05), rnd(E, F, d, scale=0.05), rnd(E, d, F, scale=0.05)
        x = rnd(T, d)
        cg = torch.Generator().manual_seed(1)
        ids = torch.stack([torch.randperm(E, generator=cg)[:k] for _ in range(T)]).int().to(dev)
        wts = torch.rand(T, k, generator=cg).to(dev)
        active = len(set(ids.flatten().tolist()))

        def fn():
            if a.torch:
                from . import reference as ref
                return ref.moe_experts(x, ids, wts, wg, wu, wd)
            y, dest = nat.moe_routed(x, ids, wts, wg, wu, wd, 0)
            return nat.moe_combine(y, dest, wts, None, None)

        ms = timeit(fn, a.iters, a.warmup)
        report(f"moe T={T} E={E} k={k} F={F} d={d}" + (" [torch]" if a.torch else ""), ms, active * 3 * F * d * 2,
               6.0 * T * k * F * d, {"active_experts": active})
    elif a.case == "attn":
        B, S, H = a.B, a.S, a.H
        bs = 64
        nb = (S + bs - 1) // bs
        layers = max(1, int(2.6e8 // (B * nb * bs * 576 * 2)) + 1)
        caches = [rnd(B * nb * bs, 576) for _ in range(layers)]
        bt = torch.arange(B * nb, dtype=torch.int32, device=dev).view(B, nb)
        sl = torch.full((B,), S, dtype=torch.int32, device=dev)
        qs = torch.arange(B + 1, dtype=torch.int32, device=dev)
        q = rnd(B, H, 576, scale=0.3)
        i = [0]

        def fn():
            c = caches[i[0] % layers]
            i[0] += 1
            if a.torch:
                from . import reference as ref
                return ref.mla_attention(q, c, bt, sl, qs, 0.1147, 512, bs)
            return nat.mla_attention(q, c, bt, sl, qs, 0.1147, 512, bs, 1)

        ms = timeit(fn, a.iters, a.warmup)
        report(f"mla decode B={B} S={S} H={H} impl={nat.ATTN_IMPL}" + (" [torch]" if a.torch else ""), ms, B * S * 576 * 2,
               2.0 * B * H * S * (576 + 512))
    elif a.case == "prefill_attn":
        # one prompt chunk of --T tokens of one sequence (nothing cached before it), --H heads of 128 + 64 / 128 dims: the
        # per-head kernel alone (K / V already expanded), and the whole op (gather + expansion GEMM + kernel)
        T, H, bs = a.T, a.H, 64
        nb = (T + bs - 1) // bs
        cache = rnd((nb + 1) * bs, 576, scale=0.5)
        bt = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).view(1, nb)
        sl = torch.tensor([T], dtype=torch.int32, device=dev)
        qs = torch.tensor([0, T], dtype=torch.int32, device=dev)
        q = rnd(T, H * 192, scale=0.5)
        w_kv_b = rnd(H * 256, 512, scale=0.05)
        meta = {"total_kv": T, "n_q_tiles": (T + 127) // 128}
        lat, kv_start = nat.kv_gather(cache, bt, sl, T, bs)
        kv = nat.gemm(lat[:, :512], w_kv_b)
        flops = 2.0 * H * (192 + 128) * T * (T + 1) / 2
        ms = timeit(lambda: nat.mha_prefill_core(q, kv, lat, kv_start, sl, qs, 0.1147, H, meta["n_q_tiles"]), a.iters, a.warmup)
        report(f"prefill attention kernel T={T} H={H} (causal FLOPs)", ms, (T * H * (192 + 128) + kv.numel() + T * 64) * 2, flops)
        ms = timeit(lambda: nat.mha_prefill(q, cache, w_kv_b, bt, sl, qs, 0.1147, H, bs, meta), a.iters, a.warmup)
        report(f"prefill attention op (gather + K/V expansion + kernel) T={T} H={H}", ms, 0, flops + 2.0 * T * 512 * H * 256)
        nat.check_status()
    elif a.case == "route":
        # router chain of one MoE layer: logits + gating + expert sort as three launches vs the one-launch kernel
        E, k, d, T = a.E, a.k, a.d, a.T
        gx = rnd(T, d)
        wr = torch.randn(E, d, device=dev, generator=g) * 0.05
        for fused in (False, True):
            nat.FUSED_ROUTE = fused

            def fn():
                ids, wts = nat.moe_gate(gx, wr, None, k, 1, 1, 1.0, False, False, 0, False, (0, E))
                return nat.moe_permute(ids, 0, E)

            ms = timeit(fn, a.iters, a.warmup)
            report(f"route T={T} E={E} k={k} d={d} " + ("one launch" if fused else "three launches"), ms, E * d * 4 + T * d * 2, 2.0 * T * E * d)
    elif a.case == "combine_norm":
        # expert combine followed by the next block's RMSNorm: two launches vs one
        k, d, T = a.k, a.d, a.T
        y = rnd(T * k, d)
        dest = torch.randperm(T * k, device=dev).int().view(T, k)
        wts = torch.rand(T, k, device=dev)
        res = rnd(T, d)
        w = torch.ones(d, device=dev)
        for fused in (False, True):
            def fn():
                if fused:
                    return nat.moe_combine(y, dest, wts, None, res, norm=(w, 1e-6))
                out = nat.moe_combine(y, dest, wts, None, res)
                return out, nat.rmsnorm(out, w, 1e-6)[0]

            ms = timeit(fn, a.iters, a.warmup)
            report(f"combine+norm T={T} k={k} d={d} " + ("one launch" if fused else "two launches"), ms, T * (k + 3) * d * 2, 0.0)
    elif a.case == "permute":
        # expert sort of a prefill chunk: one CTA vs the histogram / scan / scatter kernels
        E, k, T = a.E, a.k, a.T
        ids = torch.randint(0, E, (T, k), device=dev, dtype=torch.int32)
        for multi in (False, True):
            nat.PERMUTE_MULTI = multi
            ms = timeit(lambda: nat.moe_permute(ids, 0, E), a.iters, a.warmup)
            report(f"permute T={T} k={k} E={E} " + ("multi-CTA" if multi else "one CTA"), ms, T * k * 4 * 4, 0.0)
    elif a.case == "sample":
        # device top-k followed by the device sampler, against the host round trip it replaces (top-k values to the host)
        V, T, kk = a.N, a.T, 64
        logits = torch.randn(T, V, device=dev, generator=g)
        params = torch.tensor([[0.8, 40.0, 0.95, 0.05, 0.5]], device=dev).repeat(T, 1)

        def fn():
            v, i = nat.topk_logits(logits, kk)
            return nat.sample_topk(v, i, params)

        ms = timeit(fn, a.iters, a.warmup)
        report(f"top-k + device sampler rows={T} vocab={V}", ms, T * V * 4, 0.0)
    torch.cuda.synchronize()
    nat.check_status()


if __name__ == "__main__":
    sys.exit(main())
