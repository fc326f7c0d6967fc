"""Micro-benchmark of the row-parallel GEMM fused with its all-reduce (o_proj / down_proj under tensor parallelism)
against the same GEMM followed by a library all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29542 \
        -m jittorinfer_b200.parallel.ar_bench --model v2

For every token count T the fused path is the one the model takes: the one-shot epilogue for T <= 256 (decode), the
two-shot epilogue above (prefill).  Inputs rotate over ``--sets`` distinct weight matrices so that the weights come from
HBM, as they do inside a model.  Both paths run eagerly by default (each call then carries ~10 us of Python launch
overhead, the same for both); ``--graph`` replays the fused path as a CUDA graph.  CUDA events on the launching stream,
max over ranks.

Roofline per call and rank: the slower of (a) FLOPs at the measured bf16 GEMM rate or the weight bytes at the measured
HBM bandwidth, whichever is larger, and (b) bytes that must cross NVLink at the measured 770 GB/s per direction:
one-shot sends the fp32 tile to each of the N-1 peers; two-shot sends (N-1)/N of the fp32 tiles to their owners and
(N-1)/N of the bf16 result back out.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

# per-rank shapes of the row-parallel GEMMs: (name, N = d_model, K = local input features)
SHAPES = {"v2": [("o_proj", 5120, 2048), ("dense_down", 5120, 1536)], "lite": [("o_proj", 2048, 1024), ("dense_down", 2048, 5472)]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="v2", choices=sorted(SHAPES))
    ap.add_argument("--tokens", default="8,64,256,1024,2048")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--sets", type=int, default=6)
    ap.add_argument("--graph", action="store_true", help="replay the fused path as a CUDA graph (default: both paths eager)")
    ap.add_argument("--timeline", action="store_true",
                    help="with the timeline build of the kernels (JITTORINFER_KERNELS_SO): per shape, how long tiles wait for "
                         "each peer after their own partial is out")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from jittorinfer_b200.ops import native
    from jittorinfer_b200.parallel.comm import Communicator, FusedCommunicator
    tokens = [int(t) for t in args.tokens.split(",")]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peaks.update(json.load(f))
    except OSError:
        pass
    d_max = max(n for _, n, _ in SHAPES[args.model])
    fused = FusedCommunicator(dev, world, rank, d_max, 2 * args.sets, max_rows_large=max(tokens))
    lib = Communicator(world, rank)
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    g_same = torch.Generator(device=dev).manual_seed(7)         # the residual stream is replicated: same on every rank
    rows = []
    tl = None
    if args.timeline:
        from jittorinfer_b200.parallel.timeline import Timeline, summarize
        tl = Timeline(dev)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters / args.sets * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for name, N, K in SHAPES[args.model]:
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16, generator=g) * 0.02 for _ in range(args.sets)]
        for T in tokens:
            x = torch.randn(T, K, device=dev, dtype=torch.bfloat16, generator=g)
            res = torch.randn(T, N, device=dev, dtype=torch.bfloat16, generator=g_same)

            def run(comm):
                comm.begin_step()
                y = None
                for w in ws:
                    y = comm.linear_all_reduce(x, w, res)
                return y

            y_f, y_l = run(fused).float(), run(lib).float()
            torch.cuda.synchronize()
            native.check_status()
            err = float((y_f - y_l).abs().max())
            us_lib = timed(lambda: run(lib))
            if args.graph:
                # replay the fused calls as one CUDA graph (as the engine does for decode): device time without the Python
                # launch overhead.  The library path stays eager.
                st = torch.cuda.Stream()
                st.wait_stream(torch.cuda.current_stream())
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.stream(st):
                    run(fused)
                    torch.cuda.synchronize()
                    dist.barrier()
                    torch.cuda.synchronize()            # the barrier's own work is over: nothing of the library is in flight
                    with torch.cuda.graph(gr, stream=st, capture_error_mode="thread_local"):
                        run(fused)
                torch.cuda.synchronize()
                dist.barrier()
                us_fused = timed(gr.replay)
            else:
                if tl is not None:
                    tl.clear()
                us_fused = timed(lambda: run(fused))
            native.check_status()
            waits = None
            if tl is not None:          # every rank reads its own ring; rank 0's view is reported
                sm = summarize(tl.read())
                waits = {"wait_us_mean": round(sm.get("wait_us_mean", 0.0), 2), "dropped": tl.dropped(),
                         "late_us_by_source": {r: round(e["late_us_mean"], 2) for r, e in sm["sources"].items()}}
            flops = 2.0 * T * N * K
            t_math = max(flops / (float(peaks["bf16_tflops"]) * 1e12), N * K * 2 / (float(peaks["hbm_gbs"]) * 1e9)) * 1e6
            if T <= fused.max_rows:
                link = T * N * 4 * (world - 1)
            else:
                link = T * N * (4 + 2) * (world - 1) / world
            t_link = link / 770e9 * 1e6
            roof = max(t_math, t_link)
            rows.append({"gemm": name, "T": T, "N": N, "K": K, "path": "one-shot" if T <= fused.max_rows else "two-shot",
                         "us_library": round(us_lib, 2), "us_fused": round(us_fused, 2), "speedup": round(us_lib / us_fused, 2),
                         "roofline_us": round(roof, 2), "bound": "nvlink" if t_link > t_math else "gemm",
                         "fraction_of_roofline": round(roof / us_fused, 3), "max_abs_diff": err})
            if waits is not None:
                rows[-1]["timeline"] = waits
    if rank == 0:
        print(json.dumps({"bench": "gemm_allreduce", "model": args.model, "n_gpus": world, "timing": "CUDA events, max over ranks",
                          "fused_path": "cuda graph" if args.graph else "eager", "rows": rows}))
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
