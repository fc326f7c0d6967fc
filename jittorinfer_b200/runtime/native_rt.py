"""ctypes binding of ``libjib200_runtime.so`` (paged-KV allocator + continuous-batching scheduler).

The library is built on first use if it is missing (host C++ only, a few seconds).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import List, Optional, Tuple

import numpy as np

_lib = None
_lock = threading.Lock()

i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)


class StepArrays(C.Structure):
    _fields_ = [("tokens", i32p), ("positions", i32p), ("slot_mapping", i32p), ("q_start", i32p), ("seq_lens", i32p),
                ("seq_slots", i32p), ("block_tables", i32p), ("out_rows", i32p), ("out_slots", i32p),
                ("cap_tokens", C.c_int32), ("cap_seqs", C.c_int32), ("max_blocks_per_seq", C.c_int32)]


def lib():
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        from .. import build
        override = os.environ.get("JITTORINFER_RUNTIME_SO")      # e.g. a sanitizer-instrumented build
        path = override or build.RUNTIME_SO
        if override:
            pass
        elif not os.path.exists(path) or os.environ.get("JITTORINFER_REBUILD"):
            build.build_runtime()
        else:
            try:
                build.build_runtime()     # no-op when up to date
            except Exception:
                pass
        L = C.CDLL(path)
        vp = C.c_void_p

        def sig(name, res, *args):
            f = getattr(L, name)
            f.restype = res
            f.argtypes = list(args)

        sig("jib_kv_create", vp, C.c_int, C.c_int, C.c_int)
        sig("jib_kv_destroy", None, vp)
        sig("jib_kv_append", C.c_int, vp, C.c_int, C.c_int, i32p)
        sig("jib_kv_blocks_needed", C.c_int, vp, C.c_int, C.c_int)
        sig("jib_kv_seq_rm", C.c_int, vp, C.c_int, C.c_int, C.c_int)
        sig("jib_kv_seq_cp", C.c_int, vp, C.c_int, C.c_int, C.c_int, C.c_int)
        sig("jib_kv_seq_keep", None, vp, C.c_int)
        sig("jib_kv_clear", None, vp)
        sig("jib_kv_seq_len", C.c_int, vp, C.c_int)
        sig("jib_kv_seq_blocks", C.c_int, vp, C.c_int, i32p, C.c_int)
        for n in ("free_blocks", "used_blocks", "n_blocks", "block_size", "check"):
            sig("jib_kv_" + n, C.c_int, vp)
        sig("jib_kv_refcount", C.c_int, vp, C.c_int)
        sig("jib_kv_reserve", C.c_int, vp, C.c_int)
        sig("jib_kv_unreserve", None, vp)
        sig("jib_kv_track_freed", None, vp, C.c_int)
        sig("jib_kv_take_freed", C.c_int, vp, i32p, C.c_int)
        sig("jib_kv_fragmentation", C.c_float, vp)
        sig("jib_kv_take_copies", C.c_int, vp, i32p, i32p, C.c_int)
        sig("jib_kv_defrag", C.c_int, vp, C.c_int, i32p, i32p)
        sig("jib_sched_create", vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int)
        sig("jib_sched_destroy", None, vp)
        sig("jib_sched_add", None, vp, C.c_int64, i32p, C.c_int, C.c_int, C.c_int)
        sig("jib_sched_add_keep", None, vp, C.c_int64, i32p, C.c_int, C.c_int, C.c_int, C.c_int)
        sig("jib_sched_cancel", C.c_int, vp, C.c_int64)
        sig("jib_sched_step", C.c_int, vp, C.POINTER(StepArrays), i32p)
        sig("jib_sched_commit", None, vp, i32p, C.c_int)
        sig("jib_sched_can_run_ahead", C.c_int, vp)
        sig("jib_sched_commit_deferred", None, vp, C.c_int)
        sig("jib_sched_resolve", None, vp, i32p, C.c_int)
        sig("jib_sched_take_events", C.c_int, vp, i64p, C.c_int)
        for n in ("idle", "n_waiting", "n_running"):
            sig("jib_sched_" + n, C.c_int, vp)
        sig("jib_sched_set_n_batch", None, vp, C.c_int)
        sig("jib_sched_set_mixed_prompt_budget", None, vp, C.c_int)
        sig("jib_sched_slot_state", C.c_int, vp, C.c_int)
        sig("jib_sched_slot_cached", C.c_int, vp, C.c_int)
        sig("jib_sched_stats", None, vp, i64p)
        sig("jib_sched_out_reqs", C.c_int, vp, i64p, C.c_int)
        sig("jib_sched_slot_req", C.c_int64, vp, C.c_int)
        _lib = L
        return L


def _p32(a: np.ndarray):
    return a.ctypes.data_as(i32p)


class PagedKV:
    """Block allocator: sequences own ordered lists of fixed-size blocks (see csrc/runtime/kv_paged.h)."""

    def __init__(self, n_blocks: int, block_size: int, max_seqs: int):
        self._L = lib()
        self._h = self._L.jib_kv_create(n_blocks, block_size, max_seqs)
        self.n_blocks, self.block_size, self.max_seqs = n_blocks, block_size, max_seqs

    def __del__(self):
        try:
            if self._h:
                self._L.jib_kv_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def append(self, seq: int, n: int) -> Optional[np.ndarray]:
        out = np.empty(n, dtype=np.int32)
        return out if self._L.jib_kv_append(self._h, seq, n, _p32(out)) == 0 else None

    def blocks_needed(self, seq, n): return self._L.jib_kv_blocks_needed(self._h, seq, n)
    def seq_rm(self, seq, p0=0, p1=-1): return bool(self._L.jib_kv_seq_rm(self._h, seq, p0, p1))
    def seq_cp(self, src, dst, p0=0, p1=-1): return bool(self._L.jib_kv_seq_cp(self._h, src, dst, p0, p1))
    def seq_keep(self, seq): self._L.jib_kv_seq_keep(self._h, seq)
    def clear(self): self._L.jib_kv_clear(self._h)
    def seq_len(self, seq): return self._L.jib_kv_seq_len(self._h, seq)

    def seq_blocks(self, seq) -> np.ndarray:
        n = self._L.jib_kv_seq_blocks(self._h, seq, None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        self._L.jib_kv_seq_blocks(self._h, seq, _p32(out), n)
        return out[:n]

    @property
    def free_blocks(self): return self._L.jib_kv_free_blocks(self._h)
    @property
    def used_blocks(self): return self._L.jib_kv_used_blocks(self._h)
    def refcount(self, b): return self._L.jib_kv_refcount(self._h, b)
    def fragmentation(self): return float(self._L.jib_kv_fragmentation(self._h))
    def check(self): return bool(self._L.jib_kv_check(self._h))
    def reserve(self, n: int) -> int: return self._L.jib_kv_reserve(self._h, n)      # memory-pressure injection (tests)
    def unreserve(self) -> None: self._L.jib_kv_unreserve(self._h)

    def track_freed(self, on: bool) -> None: self._L.jib_kv_track_freed(self._h, int(on))

    def take_freed(self) -> np.ndarray:
        """Blocks whose last reference went away since the previous call and that are still free (debug poisoning)."""
        out = np.empty(self.n_blocks, dtype=np.int32)
        return out[:self._L.jib_kv_take_freed(self._h, _p32(out), out.shape[0])]

    def take_copies(self, cap: int = 4096) -> Tuple[np.ndarray, np.ndarray]:
        s = np.empty(cap, dtype=np.int32)
        d = np.empty(cap, dtype=np.int32)
        n = self._L.jib_kv_take_copies(self._h, _p32(s), _p32(d), cap)
        return s[:n], d[:n]

    def defrag(self, max_moves: int) -> Tuple[np.ndarray, np.ndarray]:
        s = np.empty(max(max_moves, 1), dtype=np.int32)
        d = np.empty(max(max_moves, 1), dtype=np.int32)
        n = self._L.jib_kv_defrag(self._h, max_moves, _p32(s), _p32(d))
        return s[:n], d[:n]


FINISH_NAMES = {0: None, 1: "stop", 2: "length", 3: "cancelled", 4: "error"}
SLOT_STATES = ("IDLE", "STARTED", "PROCESSING_PROMPT", "DONE_PROMPT", "GENERATING")


class Scheduler:
    """Continuous batching + chunked prefill (see csrc/runtime/scheduler.h).  Fills caller arrays."""

    def __init__(self, kv: PagedKV, n_slots: int, n_batch: int, n_ctx_slot: int, eos_id: int, n_keep: int = 0,
                 cont_batching: bool = True):
        self._L = lib()
        self.kv = kv
        self.n_slots = n_slots
        self._h = self._L.jib_sched_create(kv._h, n_slots, n_batch, n_ctx_slot, eos_id, n_keep, int(cont_batching))
        self._info = np.zeros(8, dtype=np.int32)
        self._ev = np.zeros(6 * 1024, dtype=np.int64)

    def __del__(self):
        try:
            if self._h:
                self._L.jib_sched_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def add(self, req_id: int, prompt, max_new: int = -1, ignore_eos: bool = False, n_keep=None):
        """``n_keep``: head tokens kept if the prompt must be cut to fit a slot (None: the scheduler's; <0: all that fits)."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        if n_keep is None:
            self._L.jib_sched_add(self._h, req_id, _p32(p), len(p), max_new, int(ignore_eos))
        else:
            self._L.jib_sched_add_keep(self._h, req_id, _p32(p), len(p), max_new, int(ignore_eos), int(n_keep))

    def cancel(self, req_id: int) -> bool:
        return bool(self._L.jib_sched_cancel(self._h, req_id))

    def step(self, arrays: StepArrays) -> np.ndarray:
        """Returns int32 info: n_tokens, n_seqs, n_out, n_decode_seqs, max_q_len, n_preempted, n_copies."""
        self._L.jib_sched_step(self._h, C.byref(arrays), _p32(self._info))
        return self._info

    def commit(self, sampled: np.ndarray, n_out: int):
        self._L.jib_sched_commit(self._h, _p32(sampled), n_out)

    # running one step ahead of the sampled ids (csrc/runtime/scheduler.h)
    def can_run_ahead(self) -> bool:
        return bool(self._L.jib_sched_can_run_ahead(self._h))

    def commit_deferred(self, n_out: int) -> None:
        self._L.jib_sched_commit_deferred(self._h, n_out)

    def resolve(self, sampled: np.ndarray, n_out: int) -> None:
        self._L.jib_sched_resolve(self._h, _p32(sampled), n_out)

    def take_events(self) -> List[Tuple[int, int, int, Optional[str], int, int]]:
        n = self._L.jib_sched_take_events(self._h, self._ev.ctypes.data_as(i64p), len(self._ev) // 6)
        ev = self._ev[: 6 * n].reshape(n, 6)
        return [(int(e[0]), int(e[1]), int(e[2]), FINISH_NAMES[int(e[3])], int(e[4]), int(e[5])) for e in ev]

    def out_reqs(self, n_out: int) -> np.ndarray:
        """Request id of each output row of the last step()."""
        o = self._ev[:max(n_out, 1)]
        n = self._L.jib_sched_out_reqs(self._h, o.ctypes.data_as(i64p), n_out)
        return o[:n].copy()

    def slot_req(self, slot: int) -> int:
        return int(self._L.jib_sched_slot_req(self._h, slot))

    def idle(self): return bool(self._L.jib_sched_idle(self._h))
    def n_waiting(self): return self._L.jib_sched_n_waiting(self._h)
    def n_running(self): return self._L.jib_sched_n_running(self._h)
    def set_n_batch(self, n): self._L.jib_sched_set_n_batch(self._h, n)
    def set_mixed_prompt_budget(self, n): self._L.jib_sched_set_mixed_prompt_budget(self._h, n)
    def slot_state(self, slot): return SLOT_STATES[self._L.jib_sched_slot_state(self._h, slot)]
    def slot_cached(self, slot): return self._L.jib_sched_slot_cached(self._h, slot)      # prompt tokens reused at launch

    def stats(self) -> dict:
        o = np.zeros(8, dtype=np.int64)
        self._L.jib_sched_stats(self._h, o.ctypes.data_as(i64p))
        return dict(zip(("steps", "prompt_tokens", "decode_tokens", "preemptions", "finished", "prefix_hits", "prefix_shared"),
                        map(int, o)))
