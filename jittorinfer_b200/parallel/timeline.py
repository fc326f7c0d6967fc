"""Device-side timeline of the in-kernel collectives: registration, read-back and analysis.

The kernels built with ``-DJIB_TIMELINE`` (``build.build_kernels_timeline()``, loaded through
``JITTORINFER_KERNELS_SO``) append ``{%globaltimer ns, kind, call site, tile, rank}`` records to a ring in device memory
(``csrc/kernels/timeline.cuh`` lists the kinds).  This module hands the ring to the library, copies it back and answers the
question a wall clock cannot: inside a fused GEMM + all-reduce, how long does a tile wait for each peer after its own
partial is out -- i.e. is the step bound by the link, by the slowest rank, or by the kernel itself?

    tl = Timeline(device)                 # registers the ring with every translation unit that stamps
    ... run a few decode steps ...
    stamps = tl.read()                    # numpy structured array, in stamping order
    print(format_summary(summarize(stamps)))

All times are on the clock of the stamping GPU; only differences between stamps of one rank are meaningful.
(The reference has no timeline: its collectives are library calls followed by a blocking stream sync,
ggml/src/ggml-cann/aclnn_ops.cpp:522-536.)
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, List

import numpy as np

STAMP_DTYPE = np.dtype([("t", "<u8"), ("kind", "<i4"), ("a", "<i4"), ("b", "<i4"), ("c", "<i4")])      # JibStamp
KIND_NAMES = {10: "oneshot_signalled", 11: "oneshot_source_arrived", 12: "oneshot_all_seen", 20: "twoshot_signalled",
              21: "twoshot_owner_source_arrived", 22: "twoshot_delivered", 30: "gemm_accumulators_done"}
UNITS = ("gemm", "comm", "combine_ar")


class Timeline:
    """Ring of ``capacity`` stamps on ``device``; needs the timeline build of the kernel library."""

    def __init__(self, device, capacity: int = 1 << 20):
        import torch

        from ..ops import native
        self.L = native.load()
        if not hasattr(self.L, "jib_timeline_enabled") or not self.L.jib_timeline_enabled():
            raise RuntimeError("the loaded kernel library has no timeline: build it with build.build_kernels_timeline() and "
                               "point JITTORINFER_KERNELS_SO at it")
        self.device = torch.device(device)
        self.capacity = int(capacity)
        self.buf = torch.zeros(self.capacity * STAMP_DTYPE.itemsize, dtype=torch.uint8, device=self.device)
        self.head = torch.zeros(1, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            for unit in UNITS:
                fn = getattr(self.L, "jib_timeline_set_" + unit)
                fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p, C.c_uint]
                if fn(self.buf.data_ptr(), self.head.data_ptr(), self.capacity) != 0:
                    raise RuntimeError(f"jib_timeline_set_{unit} failed")

    def clear(self) -> None:
        self.head.zero_()

    def read(self) -> np.ndarray:
        import torch
        torch.cuda.synchronize(self.device)
        n = min(int(self.head.item()), self.capacity)
        raw = self.buf[: n * STAMP_DTYPE.itemsize].cpu().numpy()
        return raw.view(STAMP_DTYPE).copy()

    def dropped(self) -> int:
        return max(0, int(self.head.item()) - self.capacity)

    def close(self) -> None:
        import torch
        with torch.cuda.device(self.device):
            for unit in UNITS:
                getattr(self.L, "jib_timeline_set_" + unit)(None, None, 0)


# ---- analysis (pure numpy: also runs where there is no GPU) --------------------------------------------------------------
def summarize(stamps: np.ndarray) -> Dict:
    """Per call site of the one-shot all-reduce: for every (site, tile) visit, the wait from "my partial is out" (kind 10)
    to "all sources seen" (kind 12), how late each source arrived relative to kind 10, and -- for GEMM epilogues -- the
    time from "accumulators done" (kind 30) to kind 10 (the push).  Visits are matched in stamping order per (site, tile)."""
    out: Dict = {"n_stamps": int(stamps.shape[0]), "sites": {}, "sources": {}}
    if stamps.shape[0] == 0:
        return out
    open_visit: Dict[tuple, Dict] = {}
    waits: Dict[int, List[float]] = {}
    pushes: Dict[int, List[float]] = {}
    late: Dict[int, List[float]] = {}
    last: Dict[int, List[int]] = {}
    acc_done: Dict[tuple, int] = {}
    for s in stamps:
        kind, site, tile, c, t = int(s["kind"]), int(s["a"]), int(s["b"]), int(s["c"]), int(s["t"])
        key = (site, tile)
        if kind == 30:
            acc_done[key] = t
        elif kind == 10:
            open_visit[key] = {"t0": t, "arrivals": {}}
            if key in acc_done:
                pushes.setdefault(site, []).append((t - acc_done.pop(key)) / 1e3)
        elif kind == 11 and key in open_visit:
            open_visit[key]["arrivals"][c] = t
        elif kind == 12 and key in open_visit:
            v = open_visit.pop(key)
            waits.setdefault(site, []).append((t - v["t0"]) / 1e3)
            if v["arrivals"]:
                worst = max(v["arrivals"], key=lambda r: v["arrivals"][r])
                last.setdefault(site, []).append(worst)
                for r, ta in v["arrivals"].items():
                    late.setdefault(r, []).append(max(0, ta - v["t0"]) / 1e3)
    for site in sorted(waits):
        w = np.asarray(waits[site])
        entry = {"visits": int(w.size), "wait_us_mean": float(w.mean()), "wait_us_p50": float(np.percentile(w, 50)),
                 "wait_us_p99": float(np.percentile(w, 99)), "wait_us_max": float(w.max())}
        if site in pushes:
            entry["push_us_mean"] = float(np.mean(pushes[site]))
        if site in last:
            ranks, counts = np.unique(np.asarray(last[site]), return_counts=True)
            entry["last_source"] = {int(r): int(n) for r, n in zip(ranks, counts)}
        out["sites"][site] = entry
    for r in sorted(late):
        a = np.asarray(late[r])
        out["sources"][r] = {"arrivals": int(a.size), "late_us_mean": float(a.mean()), "late_us_p99": float(np.percentile(a, 99))}
    all_w = np.concatenate([np.asarray(v) for v in waits.values()]) if waits else np.zeros(0)
    if all_w.size:
        out["wait_us_mean"] = float(all_w.mean())
        out["wait_us_total"] = float(all_w.sum())
    return out


def format_summary(summary: Dict, top: int = 12) -> str:
    lines = [f"{summary['n_stamps']} stamps; mean wait after signalling {summary.get('wait_us_mean', 0.0):.2f} us"]
    lines.append(f"{'source':>6s} {'arrivals':>9s} {'late mean us':>13s} {'late p99 us':>12s}")
    for r, e in summary["sources"].items():
        lines.append(f"{r:6d} {e['arrivals']:9d} {e['late_us_mean']:13.2f} {e['late_us_p99']:12.2f}")
    lines.append(f"{'site':>6s} {'visits':>7s} {'wait mean':>10s} {'p50':>8s} {'p99':>8s} {'max':>8s} {'push mean':>10s}  last source (count)")
    ranked = sorted(summary["sites"].items(), key=lambda kv: -kv[1]["wait_us_mean"])[:top]
    for site, e in ranked:
        lines.append(f"{site:6d} {e['visits']:7d} {e['wait_us_mean']:10.2f} {e['wait_us_p50']:8.2f} {e['wait_us_p99']:8.2f} "
                     f"{e['wait_us_max']:8.2f} {e.get('push_us_mean', float('nan')):10.2f}  {e.get('last_source', {})}")
    return "\n".join(lines)


def to_chrome_trace(stamps: np.ndarray, rank: int = 0) -> str:
    """Instant events for chrome://tracing / Perfetto: one process per rank, one thread row per call site."""
    t0 = int(stamps["t"].min()) if stamps.shape[0] else 0
    ev = [{"name": KIND_NAMES.get(int(s["kind"]), str(int(s["kind"]))), "ph": "i", "s": "t", "pid": rank, "tid": int(s["a"]),
           "ts": (int(s["t"]) - t0) / 1e3, "args": {"tile": int(s["b"]), "rank": int(s["c"])}} for s in stamps]
    return json.dumps({"traceEvents": ev, "displayTimeUnit": "ns"})
