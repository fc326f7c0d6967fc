"""Per-op device-time breakdown of a forward pass, without an external profiler.

``OpProfile`` temporarily wraps the functions of the ``ops`` front-end (and, when given, the methods of a communicator
or dispatcher object) so that every call is bracketed by two CUDA events on the current stream (``time.perf_counter``
for CPU tensors).  After the region the events are read once and aggregated by op name and operand shapes::

    with OpProfile(extra=[(model.comm, ("all_reduce", "linear_all_reduce"))]) as prof:
        engine.step()                      # eager step (a captured graph replays kernels without passing through ops)
    print(prof.format())

Events bracket the op on its stream, so for large (prefill) batches the numbers are kernel times; for decode-sized
batches, where the host launches slower than the device executes, an op's time includes the wait for its launch and
the table shows where the *step* goes rather than what the kernels cost.  Nested ops (``moe_ffn`` calling
``moe_experts``) are reported at the outermost level only.

Command line (random-init weights; one prefill chunk and a few eager decode steps)::

    python -m jittorinfer_b200.ops.profile --model lite --prefill 2048 --decode-batch 8 --json breakdown.json
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m jittorinfer_b200.ops.profile --model v2

(under ``torchrun`` the model is tensor/expert-parallel over the ranks, the collectives appear as rows of their own, and
rank 0 prints its view).

This is the counterpart of the reference's per-op timing helpers (``llama_perf_context`` gives totals only; its op-speed
test times single ops: tests/test_ops_speed.cpp).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

OPS = ("embed_gather", "select_rows", "rmsnorm", "linear", "gateup_silu", "mla_qkv_post", "q_absorb", "v_up", "mla_attention",
       "moe_gate", "moe_experts", "moe_ffn", "argmax", "topk_logits", "sample_topk", "kv_block_copy")


def _sig(args, kwargs) -> str:
    shapes = []
    for a in list(args) + list(kwargs.values()):
        if isinstance(a, torch.Tensor) and a.dim() > 0:
            shapes.append("x".join(str(int(s)) for s in a.shape))
        if len(shapes) == 3:
            break
    return " ".join(shapes)


KERNEL_LEVEL = ("gemm", "gemm_batched", "gemm_grouped_raw", "moe_permute", "gather_rows", "moe_combine", "rmsnorm", "embed_gather",
                "mla_qkv_post", "mla_attention", "moe_gate", "argmax", "topk_logits", "kv_block_copy", "mha_prefill", "kv_gather",
                "mha_prefill_core")


class OpProfile:
    """``leaves=True`` also wraps the kernel-level functions of ``ops.native`` and reports only the innermost timed
    calls, labelled with their path (``moe_ffn/gemm_grouped_raw``): the breakdown inside the composite ops."""

    def __init__(self, extra: Iterable[Tuple[object, Sequence[str]]] = (), names: Sequence[str] = OPS, leaves: bool = False):
        self.names = tuple(names)
        self.leaves = leaves
        self.extra = [(obj, tuple(meths)) for obj, meths in extra if obj is not None]
        self.records: List[Tuple[str, str, object, object]] = []      # name, signature, start, end (events or floats)
        self._saved: List[Tuple[object, str, object, bool]] = []
        self._stack: List[List] = []                                   # open calls: [label, has_timed_child]
        self.rows: List[Dict] = []
        self.total_ms = 0.0
        self.wall_ms = 0.0

    # ---- wrapping ----------------------------------------------------------------------------------------------
    def _wrap(self, label: str, fn):
        def wrapped(*args, **kwargs):
            if self._stack and not self.leaves:       # inner op of an op that is already being timed
                return fn(*args, **kwargs)
            cuda = any(isinstance(a, torch.Tensor) and a.is_cuda for a in list(args) + list(kwargs.values()))
            if not cuda and self.leaves and torch.cuda.is_available():
                cuda = True                           # kernel-level functions that take raw pointers
            if self._stack:
                self._stack[-1][1] = True
            frame = [label if not self._stack else self._stack[-1][0] + "/" + label, False]
            self._stack.append(frame)
            try:
                if cuda:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = fn(*args, **kwargs)
                    e1.record()
                else:
                    e0 = time.perf_counter()
                    out = fn(*args, **kwargs)
                    e1 = time.perf_counter()
            finally:
                self._stack.pop()
            if not frame[1]:                          # a call that contained timed calls is the sum of those
                self.records.append((frame[0], _sig(args, kwargs), e0, e1))
            return out
        wrapped.__wrapped__ = fn
        return wrapped

    def __enter__(self):
        from .. import ops
        for n in self.names:
            fn = getattr(ops, n, None)
            if fn is not None:
                self._saved.append((ops, n, fn, True))
                setattr(ops, n, self._wrap(n, fn))
        if self.leaves and torch.cuda.is_available():
            native = ops.nat()
            for n in KERNEL_LEVEL:
                fn = getattr(native, n, None)
                if fn is not None:
                    self._saved.append((native, n, fn, True))
                    setattr(native, n, self._wrap(n, fn))
        for obj, meths in self.extra:
            for m in meths:
                fn = getattr(obj, m, None)
                if fn is None:
                    continue
                had = m in getattr(obj, "__dict__", {})
                self._saved.append((obj, m, obj.__dict__.get(m) if had else None, had))
                setattr(obj, m, self._wrap(type(obj).__name__ + "." + m, fn))
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        for obj, n, fn, had in reversed(self._saved):
            if had:
                setattr(obj, n, fn)
            else:
                delattr(obj, n)                       # the instance attribute shadowed a class method: uncover it
        self._saved.clear()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.wall_ms = (time.perf_counter() - self._t0) * 1e3
        self._aggregate()
        return False

    # ---- results -----------------------------------------------------------------------------------------------
    def _aggregate(self) -> None:
        agg: Dict[Tuple[str, str], List[float]] = {}
        for name, sig, e0, e1 in self.records:
            ms = e0.elapsed_time(e1) if not isinstance(e0, float) else (e1 - e0) * 1e3
            a = agg.setdefault((name, sig), [0, 0.0])
            a[0] += 1
            a[1] += ms
        self.total_ms = sum(v[1] for v in agg.values())
        self.rows = [{"op": k[0], "shapes": k[1], "calls": v[0], "total_ms": v[1], "ms_per_call": v[1] / v[0],
                      "share": v[1] / self.total_ms if self.total_ms > 0 else 0.0}
                     for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])]

    def by_op(self) -> List[Dict]:
        agg: Dict[str, List[float]] = {}
        for r in self.rows:
            a = agg.setdefault(r["op"], [0, 0.0])
            a[0] += r["calls"]
            a[1] += r["total_ms"]
        return [{"op": k, "calls": v[0], "total_ms": v[1], "share": v[1] / self.total_ms if self.total_ms > 0 else 0.0}
                for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])]

    def format(self, top: int = 30) -> str:
        lines = [f"ops {self.total_ms:.3f} ms in {len(self.records)} calls; wall {self.wall_ms:.3f} ms",
                 f"{'op':40s} {'calls':>6s} {'total ms':>10s} {'share':>7s}"]
        for r in self.by_op():
            lines.append(f"{r['op']:40s} {r['calls']:6d} {r['total_ms']:10.3f} {100 * r['share']:6.1f}%")
        lines.append("")
        lines.append(f"{'op':40s} {'calls':>6s} {'ms/call':>9s} {'share':>7s}  shapes")
        for r in self.rows[:top]:
            lines.append(f"{r['op']:40s} {r['calls']:6d} {r['ms_per_call']:9.4f} {100 * r['share']:6.1f}%  {r['shapes']}")
        return "\n".join(lines)

    def to_json(self) -> Dict:
        return {"total_ms": self.total_ms, "wall_ms": self.wall_ms, "n_calls": len(self.records), "by_op": self.by_op(),
                "rows": self.rows}


def comm_hooks(model) -> List[Tuple[object, Sequence[str]]]:
    """The collective entry points of a model's communicator / expert dispatcher, for ``OpProfile(extra=...)``."""
    return [(getattr(model, "comm", None), ("all_reduce", "linear_all_reduce", "all_gather_rows", "allgather_linear",
                                            "reduce_scatter_rows", "linear_reduce_scatter", "moe_ffn_all_reduce")),
            (getattr(model, "ep", None), ("moe_ffn",))]


def profile_engine(engine, prefill_tokens: int, decode_batch: int, decode_steps: int = 4, seed: int = 0,
                   leaves: bool = False) -> Dict[str, OpProfile]:
    """One prefill chunk of ``prefill_tokens`` (one sequence) and ``decode_steps`` eager decode steps of ``decode_batch``
    sequences.  The engine must have been built with ``cuda_graphs=False`` for the decode part to pass through ``ops``."""
    from ..runtime.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    n_vocab = engine.hp.n_vocab
    out: Dict[str, OpProfile] = {}
    extra = comm_hooks(engine.model)
    sp = SamplingParams(ignore_eos=True, max_tokens=decode_steps + 8)
    ahead = engine.set_run_ahead(False)            # every profiled step() must contain its own forward pass
    if prefill_tokens > 0:
        warm = engine.add_request(torch.randint(0, n_vocab, (prefill_tokens,), generator=g).tolist(), sp)      # untimed: first-call costs
        engine.step()
        engine.cancel(warm)
        rid = engine.add_request(torch.randint(0, n_vocab, (prefill_tokens,), generator=g).tolist(), sp)
        with OpProfile(extra=extra, leaves=leaves) as prof:
            engine.step()
        out["prefill"] = prof
        engine.cancel(rid)
        while engine.has_work():
            engine.step()
    if decode_batch > 0:
        rids = [engine.add_request(torch.randint(0, n_vocab, (16,), generator=g).tolist(), sp) for _ in range(decode_batch)]
        engine.step()                                  # prompts
        engine.step()                                  # first decode step, untimed
        with OpProfile(extra=extra, leaves=leaves) as prof:
            for _ in range(decode_steps):
                engine.step()
        out["decode"] = prof
        for r in rids:
            engine.cancel(r)
    engine.set_run_ahead(ahead)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="lite", help="hyper-parameter preset (tiny, lite, v2, ...)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the profiled prefill chunk (0 = skip)")
    ap.add_argument("--decode-batch", type=int, default=8, help="sequences of the profiled decode steps (0 = skip)")
    ap.add_argument("--decode-steps", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="keep only this many layers (0 = all): a smaller model of the same shapes")
    ap.add_argument("--leaves", action="store_true", help="break composite ops down to their kernel-level calls")
    ap.add_argument("--json", default=None, help="write the tables to this file")
    args = ap.parse_args(argv)
    import dataclasses

    from ..models.hparams import preset
    from ..runtime.factory import build_engine
    hp = preset(args.model)
    if args.layers:
        hp = dataclasses.replace(hp, n_layer=args.layers, n_layer_dense_lead=min(hp.n_layer_dense_lead, args.layers))
    # under torchrun (WORLD_SIZE > 1) the model is tensor/expert-parallel over the ranks; rank 0 reports its own view
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device(args.device)
    if world > 1:
        import torch.distributed as dist
        if dev.type == "cuda":
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    n_slot = max(args.prefill + 64, 256)
    eng = build_engine(hp, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, world=world, rank=rank,
                       n_parallel=max(args.decode_batch, 1) + 2, n_ctx_slot=n_slot, n_batch=max(args.prefill, 64),
                       cuda_graphs=False)
    res = profile_engine(eng, args.prefill, args.decode_batch, args.decode_steps, leaves=args.leaves)
    if rank == 0:
        for phase, prof in res.items():
            print(f"== {phase} ==")
            print(prof.format())
            print()
    if world > 1:
        dist.barrier()
        if rank != 0:
            return 0
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"model": args.model, "layers": hp.n_layer, "prefill_tokens": args.prefill, "decode_batch": args.decode_batch,
                       "decode_steps": args.decode_steps, **{k: v.to_json() for k, v in res.items()}}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
