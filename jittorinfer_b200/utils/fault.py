"""Host-side fault injection.

``JITTORINFER_FAULT="site:n[,site:n...]"`` makes the n-th pass (1-based) through the named site fail; ``site:n+``
fails the n-th and every later pass.  Sites are plain strings checked with ``fault.check(site)`` in host code:

=================  ==================================================================================
``kv_alloc``       the scheduler's step: the KV allocator reports "no blocks" (slot preemption path)
``engine_step``    ``LLMEngine.step`` raises before launching anything (server: fail in-flight requests, keep serving)
``gguf_read``      the GGUF reader raises on open (server start / model load error path)
``transport``      the rank-0 task broadcast raises (multi-rank control plane)
``heartbeat``      a worker stops publishing heartbeats (failure detector)
=================  ==================================================================================

Nothing here touches a GPU: device-side waits are bounded and report through status words, and their timeout path is
exercised by withholding a flag, never by a trap or an endless loop.  The reference has no failure handling at all: any
ACL/HCCL error aborts the process (ggml/src/ggml-cann/common.h:73-85) and worker ranks block forever in ``MPI_Bcast`` if
rank 0 dies (examples/mpi_server/server.cpp:1896-1898).
"""
from __future__ import annotations

import os
import threading
from typing import Dict, Tuple


class InjectedFault(RuntimeError):
    """Raised by ``check`` at an armed site."""


_lock = threading.Lock()
_plan: Dict[str, Tuple[int, bool]] = {}
_count: Dict[str, int] = {}


def configure(spec: str = "") -> None:
    """(Re)arm from a spec string; an empty spec disarms everything."""
    with _lock:
        _plan.clear()
        _count.clear()
        for item in filter(None, (s.strip() for s in spec.split(","))):
            site, _, n = item.partition(":")
            sticky = n.endswith("+")
            _plan[site] = (int(n.rstrip("+") or 1), sticky)


def armed(site: str) -> bool:
    return site in _plan


def hit(site: str) -> bool:
    """Counts a pass through ``site``; True if this pass must fail."""
    if not _plan:
        return False
    with _lock:
        if site not in _plan:
            return False
        _count[site] = _count.get(site, 0) + 1
        n, sticky = _plan[site]
        return _count[site] == n or (sticky and _count[site] > n)


def check(site: str) -> None:
    if hit(site):
        raise InjectedFault(f"injected fault at {site} (pass {_count.get(site)})")


configure(os.environ.get("JITTORINFER_FAULT", ""))
