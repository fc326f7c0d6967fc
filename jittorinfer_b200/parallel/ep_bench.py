"""Micro-benchmark of one expert-parallel MoE layer (dispatch + grouped expert GEMMs + combine) with data-parallel
tokens: the fused peer-memory path against the library all-to-all path.

Launch one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \
        -m jittorinfer_b200.parallel.ep_bench --tokens 64 --model lite

Every rank holds ``--tokens`` tokens (uniform random routing), ``n_expert / N`` experts.  The timed region is
``--layers`` consecutive MoE layers (distinct call sites, distinct weights so that every layer streams its expert
weights from HBM), repeated ``--iters`` times; CUDA events on the launching stream, max over ranks.  The fused path is
replayed as one CUDA graph; the library path cannot be captured (it reads split sizes on the host) and runs eagerly.

Roofline per layer and rank: the slower of (a) expert weights that must be streamed from HBM at the measured copy
bandwidth and (b) bytes that must cross NVLink (rows out and results back, the share that goes to other ranks) at the
measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

SHAPES = {"lite": dict(E=64, d=2048, F=1408, k=6), "v2": dict(E=160, d=5120, F=1536, k=6)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="lite", choices=sorted(SHAPES))
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from jittorinfer_b200.ops import native
    from jittorinfer_b200.parallel.ep import EpDispatcher, FusedEpDispatcher
    sh = SHAPES[args.model]
    E, d, F, k, T = sh["E"], sh["d"], sh["F"], sh["k"], args.tokens
    El = E // world
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    weights = [(torch.randn(El, F, d, device=dev, dtype=torch.bfloat16, generator=g) * 0.02,
                torch.randn(El, F, d, device=dev, dtype=torch.bfloat16, generator=g) * 0.02,
                torch.randn(El, d, F, device=dev, dtype=torch.bfloat16, generator=g) * 0.02) for _ in range(args.layers)]
    x = torch.randn(T, d, device=dev, dtype=torch.bfloat16, generator=g)
    scores = torch.rand(T, E, device=dev, generator=g)
    ids = scores.topk(k, dim=1).indices.int().contiguous()
    wts = torch.full((T, k), 1.0 / k, device=dev, dtype=torch.float32)

    def step(ep):
        ep.begin_step()
        y = x
        for wg, wu, wd in weights:
            y = ep.moe_ffn(x, None, ids, wts, wg, wu, wd, None)
        return y

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters / args.layers * 1e3], device=dev)     # us per layer
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    lib = EpDispatcher(world, rank, E)
    y_lib = step(lib)
    us_lib = timed(lambda: step(lib))

    fused = FusedEpDispatcher(dev, world, rank, E, d, k, args.layers, max_tokens=max(T, 1))
    y_fused = step(fused)
    torch.cuda.synchronize()
    native.check_status()
    err = float((y_fused.float() - y_lib.float()).abs().max())
    us_eager = timed(lambda: step(fused))
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step(fused)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()                        # the barrier's own work is over: nothing of the library is in flight
        with torch.cuda.graph(graph, stream=s, capture_error_mode="thread_local"):
            step(fused)
    torch.cuda.synchronize()
    dist.barrier()
    us_graph = timed(graph.replay)
    native.check_status()

    peaks = {"hbm_gbs": 6650.0}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")) as f:
            peaks.update(json.load(f))
    except OSError:
        pass
    # experts a rank touches: all of its local ones once T*k*world >> E_local (the benchmark's regime)
    touched = min(El, T * k * world)
    w_bytes = touched * 3 * F * d * 2
    link_bytes = T * k * d * 2 * (world - 1) / world                  # one direction; the return is the same size the other way
    t_hbm = w_bytes / (float(peaks["hbm_gbs"]) * 1e9) * 1e6
    t_link = link_bytes / 770e9 * 1e6
    roof = max(t_hbm, t_link)
    if rank == 0:
        print(json.dumps({"bench": "ep_moe_layer", "model": args.model, "n_gpus": world, "tokens_per_rank": T, "layers": args.layers,
                          "us_per_layer": {"library_all_to_all": round(us_lib, 2), "fused_eager": round(us_eager, 2),
                                           "fused_graph": round(us_graph, 2)},
                          "speedup_vs_library": round(us_lib / us_graph, 2), "max_abs_diff_vs_library": err,
                          "roofline_us": {"hbm_weights": round(t_hbm, 2), "nvlink_rows": round(t_link, 2)},
                          "fraction_of_roofline": round(roof / us_graph, 3), "timing": "CUDA events, max over ranks"}))
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
