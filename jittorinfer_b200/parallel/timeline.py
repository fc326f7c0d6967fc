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
UNITS = ("gemm", "comm", "combine_ar", "elementwise", "moe", "attn", "flash")


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


# ---- kernel phase stamps (kinds 100 + kernel id) ---------------------------------------------------------------------
KERNEL_NAMES = {1: "gemm", 2: "mla_flash", 3: "mla_combine", 4: "rmsnorm", 5: "mla_qkv_post", 6: "embed_gather", 7: "gather_rows",
                8: "argmax", 9: "router_logits", 10: "moe_gate", 11: "moe_permute", 12: "moe_combine", 13: "moe_combine_norm",
                14: "moe_route_fused", 15: "topk"}


def kernel_launches(stamps: np.ndarray) -> List[Dict]:
    """Groups the phase stamps (kind >= 100) into launches, in launch order.

    Every CTA stamps phase 0 on entry, and a kernel's CTAs all enter before the next kernel's do, so the entry stamps
    sorted by time fall into consecutive runs of ``b`` (grid size) stamps of one kind: one run per launch.  The other
    phases of a CTA are matched to its launch by counting: the n-th phase-p stamp of (kind, grid size, block) belongs to the
    n-th launch with that kind and grid size.  Per launch: name, grid, and per phase the first and last time a CTA reached
    it, in microseconds from the first entry stamp of the whole record."""
    # (launches of one kind and grid size are told apart by the order of their entry stamps per CTA)
    ks = stamps[stamps["kind"] >= 100]
    if ks.shape[0] == 0:
        return []
    ks = ks[np.argsort(ks["t"], kind="stable")]
    t0 = int(ks["t"][0])
    entries = ks[ks["c"] == 0]
    launches: List[Dict] = []
    by_key: Dict[tuple, List[int]] = {}
    # launches of one (kernel, grid size) enter in launch order even when kernels of different kinds are resident together
    # (programmatic dependent launch makes a chain of kernels resident early): chunk each kind's entry stamps by grid size
    per_key: Dict[tuple, List[int]] = {}
    for i in range(entries.shape[0]):
        per_key.setdefault((int(entries["kind"][i]), int(entries["b"][i])), []).append(int(entries["t"][i]))
    protos = []
    for (kind, grid), ts in per_key.items():
        for j in range(0, len(ts), max(1, grid)):
            chunk = ts[j:j + max(1, grid)]
            protos.append((chunk[0], kind, grid, len(chunk), chunk[-1]))
    protos.sort()
    for first, kind, grid, n_in, last in protos:
        rec = {"kernel": KERNEL_NAMES.get(kind - 100, str(kind - 100)), "grid": grid, "n_entered": n_in,
               "phases": {0: [(first - t0) / 1e3, (last - t0) / 1e3]}}
        by_key.setdefault((kind, grid), []).append(len(launches))
        launches.append(rec)
    # a later stamp of a CTA belongs to the launch whose entry stamp of that CTA is the last one before it (CTAs that leave
    # early stamp no further phases, so counting stamps per CTA would drift)
    entry_t: Dict[tuple, List[int]] = {}
    for i in range(entries.shape[0]):
        entry_t.setdefault((int(entries["kind"][i]), int(entries["b"][i]), int(entries["a"][i])), []).append(int(entries["t"][i]))
    import bisect
    for s in ks[ks["c"] != 0]:
        key = (int(s["kind"]), int(s["b"]))
        times = entry_t.get((key[0], key[1], int(s["a"])))
        idx = by_key.get(key)
        if times is None or idx is None:
            continue
        n = bisect.bisect_right(times, int(s["t"])) - 1
        if n < 0 or n >= len(idx):
            continue
        ph = launches[idx[n]]["phases"]
        t = (int(s["t"]) - t0) / 1e3
        cur = ph.get(int(s["c"]))
        if cur is None:
            ph[int(s["c"])] = [t, t]
        else:
            cur[0], cur[1] = min(cur[0], t), max(cur[1], t)
    return launches


def format_kernel_launches(launches: List[Dict]) -> str:
    """One line per launch: when its first CTA entered, when its CTAs got past the wait for the previous kernel, when the
    last CTA left, and (GEMM / attention) the kernel-specific phases as first..last over the CTAs."""
    lines = [f"{'#':>4s} {'kernel':18s} {'grid':>5s} {'enter':>9s} {'past wait':>17s} {'exit (last)':>11s} {'busy us':>8s}  other phases (first..last)"]
    prev_exit = 0.0
    for n, r in enumerate(launches):
        ph = r["phases"]
        enter = ph[0][0]
        wait = ph.get(1)
        ex = ph.get(9, [float("nan"), float("nan")])[1]
        start = wait[0] if wait else enter
        extra = "  ".join(f"p{p}:{v[0]:.1f}..{v[1]:.1f}" for p, v in sorted(ph.items()) if p not in (0, 1, 9))
        lines.append(f"{n:4d} {r['kernel']:18s} {r['grid']:5d} {enter:9.1f} {(f'{wait[0]:.1f}..{wait[1]:.1f}' if wait else '-'):>17s} {ex:11.1f} "
                     f"{ex - max(start, prev_exit):8.1f}  {extra}")
        if ex == ex:
            prev_exit = max(prev_exit, ex)
    return "\n".join(lines)
