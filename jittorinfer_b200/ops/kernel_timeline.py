"""In-graph timeline of one decode step, kernel by kernel, from device time stamps.

A profiler serialises kernels and flushes caches between them, so it cannot show what a kernel costs *inside* a replayed
CUDA graph, where launches overlap (programmatic dependent launch) and caches stay warm.  The timeline build of the kernel
library (``build.build_kernels_timeline()``) makes every CTA stamp ``%globaltimer`` on entry, once it is past the wait for
the previous kernel, at kernel-specific points and on exit; this tool replays one captured decode step with the stamps on
and prints one line per launch (``parallel/timeline.py:kernel_launches``)::

    JITTORINFER_KERNELS_SO=$(python -c "from jittorinfer_b200 import build; print(build.build_kernels_timeline())") \\
        python -m jittorinfer_b200.ops.kernel_timeline --model lite --layers 4 --batch 8 --context 1024

The stamps cost time (one atomic and one 24-byte store per CTA and phase): read the table for where a step's time goes,
not for absolute throughput.  The reference has no counterpart (it times whole ops with host clocks, tests/test_ops_speed.cpp).
"""
from __future__ import annotations

import argparse
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="lite")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=3, help="replays recorded; the last one is printed")
    ap.add_argument("--out", default=None, help="also write the table to this file")
    ap.add_argument("--raw", default=None, help="also save the last step's stamps (numpy structured array, .npy)")
    args = ap.parse_args(argv)

    from ..models.hparams import preset
    from ..parallel.timeline import Timeline, format_kernel_launches, kernel_launches
    from ..runtime.factory import build_engine
    from ..runtime.sampling import SamplingParams

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hp = preset(args.model).replace(n_layer=args.layers)
    C = args.batch
    eng = build_engine(hp, device=dev, n_parallel=C, n_ctx_slot=args.context + 128, n_batch=2048, seed=0, graph_buckets=(C,))
    g = torch.Generator().manual_seed(1)
    sp = SamplingParams(max_tokens=64, ignore_eos=True)
    ids = [eng.add_request(torch.randint(0, hp.n_vocab, (args.context,), generator=g).tolist(), sp) for _ in range(C)]
    while any(len(eng.requests[i].output) == 0 for i in ids):
        eng.step()
    for _ in range(4):
        eng.step()
    tl = Timeline(dev, capacity=1 << 20)
    text = ""
    for _ in range(args.steps):
        torch.cuda.synchronize()
        tl.clear()
        eng.step()
        stamps = tl.read()
        launches = kernel_launches(stamps)
        text = format_kernel_launches(launches)
    tl.close()
    head = f"# {args.model}, {args.layers} layers, batch {C}, context {args.context}: {len(launches)} launches in the last step"
    print(head)
    print(text)
    if args.raw:
        import numpy as np
        np.save(args.raw, stamps)
    if args.out:
        with open(args.out, "w") as f:
            f.write(head + "\n" + text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
