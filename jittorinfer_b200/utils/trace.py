"""Tracing: a per-step JSON-lines trace of the scheduler / engine, NVTX ranges, and the load-time tensor listing.

The reference has wall-clock accumulators only (``llama_perf_context``, src/llama.cpp:29-66), a tensor listing behind
``LLAMA_TRACE`` (src/llama-model-loader.cpp:491-494) and a per-layer graph dump behind ``LLAMA_PRINT_LAYER``
(src/llama-context-load-utils.cpp:154-162); it has no trace file.  Here:

* ``JITTORINFER_TRACE=<path>``: the engine appends one JSON object per step -- step number, wall time, tokens in/out,
  sequences, graph bucket or eager, KV blocks in use, fragmentation, queue depth, the host time of each phase
  (schedule / upload+launch / wait+download / commit).  ``Tracer.read`` parses a file back.
* ``JITTORINFER_NVTX=1``: ``range(name)`` pushes NVTX ranges (per forward pass and per layer) that ``ncu`` / Nsight
  show; otherwise it costs one attribute lookup.
* ``LLAMA_TRACE=1`` / ``JITTORINFER_TRACE_LOAD=1``: ``log_tensor`` prints every tensor (name, shape, dtype, shard) as it
  is placed on the device.
"""
from __future__ import annotations

import contextlib
import json
import os
import sys
import threading
import time
from typing import Any, Dict, Iterator, List, Optional

_NVTX = os.environ.get("JITTORINFER_NVTX", "") not in ("", "0")
_LOAD = os.environ.get("LLAMA_TRACE", "") not in ("", "0") or os.environ.get("JITTORINFER_TRACE_LOAD", "") not in ("", "0")


class Tracer:
    """Append-only JSON-lines writer; thread-safe; a no-op when no path is configured."""

    def __init__(self, path: Optional[str] = None):
        self.path = path if path is not None else os.environ.get("JITTORINFER_TRACE") or None
        self._f = open(self.path, "a", buffering=1) if self.path else None
        self._lock = threading.Lock()
        self.t0 = time.perf_counter()

    @property
    def enabled(self) -> bool:
        return self._f is not None

    def emit(self, kind: str, **fields: Any) -> None:
        if self._f is None:
            return
        rec = {"kind": kind, "t_ms": round((time.perf_counter() - self.t0) * 1e3, 3)}
        rec.update(fields)
        with self._lock:
            self._f.write(json.dumps(rec, separators=(",", ":")) + "\n")

    def close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None

    @staticmethod
    def read(path: str) -> List[Dict[str, Any]]:
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]


class PhaseTimer:
    """Host-side phase clock for one step: ``mark(name)`` closes the phase that was running."""

    def __init__(self):
        self.t = time.perf_counter()
        self.ms: Dict[str, float] = {}

    def mark(self, name: str) -> None:
        now = time.perf_counter()
        self.ms[name] = round(self.ms.get(name, 0.0) + (now - self.t) * 1e3, 4)
        self.t = now


@contextlib.contextmanager
def range(name: str) -> Iterator[None]:   # noqa: A001 - mirrors the NVTX vocabulary
    """NVTX range when JITTORINFER_NVTX is set and a GPU is present."""
    if not _NVTX:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_enabled() -> bool:
    return _NVTX


def log_tensor(name: str, shape, dtype, shard: str = "") -> None:
    if _LOAD:
        sys.stderr.write(f"load_tensor: {name:48s} {str(tuple(shape)):28s} {str(dtype):16s} {shard}\n")
