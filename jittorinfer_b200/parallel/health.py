"""Failure detection for multi-process serving: heartbeats through the rendezvous store.

The reference has none: worker ranks block forever in ``MPI_Bcast`` if rank 0 dies and any device error aborts the
process (examples/mpi_server/server.cpp:1896-1898; ggml/src/ggml-cann/common.h:73-85).  Here every rank runs a small
thread that writes ``hb/<rank> = <monotonic counter>`` into a ``torch.distributed`` store (TCPStore / FileStore /
HashStore) every ``interval`` seconds; any rank can ask which peers have stopped advancing for longer than ``timeout``.

Use:
* rank 0 (the HTTP front-end) checks ``dead()`` before broadcasting a step; if a worker is gone it fails the in-flight
  requests with HTTP 503 and stops instead of entering a collective that can never complete;
* workers check that rank 0 is alive while they wait for work and exit cleanly when it is not.

A rank leaves only between steps (no kernels or collectives of its own in flight), and the others learn of it here,
on the host, before their next launch -- nothing about this path needs (or is allowed to cause) a GPU fault.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

from ..utils import fault


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.2, timeout: float = 2.0, prefix: str = "hb"):
        self.store, self.rank, self.world = self._own_connection(store), rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._beat = 0
        self._seen: Dict[int, tuple] = {}          # rank -> (last counter, local time it changed)
        self.publish()

    @staticmethod
    def _own_connection(store):
        """A TCPStore client serialises its requests on one socket, so a blocking ``wait`` elsewhere in the process would
        also block the heartbeats: the detector talks to the server over a connection of its own."""
        try:
            import torch.distributed as dist
            if isinstance(store, dist.TCPStore):
                return dist.TCPStore(store.host, store.port, None, False, wait_for_workers=False)
        except Exception:
            pass
        return store

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def publish(self) -> None:
        if fault.armed("heartbeat") and fault.hit("heartbeat"):
            self._stop.set()                       # injected: this rank goes silent from now on
            return
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.publish()
                except Exception:
                    return                         # the store is gone: the job is being torn down
        self._thread = threading.Thread(target=loop, name=f"heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def _counter(self, r: int) -> Optional[int]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return int(self.store.get(self._key(r)))
        except Exception:
            return None

    def dead(self, ranks: Optional[List[int]] = None) -> List[int]:
        """Ranks whose counter has not advanced for ``timeout`` seconds (never-seen ranks count from the first look)."""
        now = time.monotonic()
        out = []
        for r in (ranks if ranks is not None else range(self.world)):
            if r == self.rank:
                continue
            c = self._counter(r)
            last = self._seen.get(r)
            if last is None or (c is not None and c != last[0]):
                self._seen[r] = (c, now)
                continue
            if now - last[1] > self.timeout:
                out.append(r)
        return out

    def wait_all_alive(self, deadline: float = 30.0) -> bool:
        """Rendezvous check at start-up: every rank has published at least once before ``deadline`` seconds pass."""
        t0 = time.monotonic()
        while time.monotonic() - t0 < deadline:
            if all(self._counter(r) is not None for r in range(self.world)):
                return True
            time.sleep(min(self.interval, 0.05))
        return False


class Watchdog:
    """Background check that the given ranks are still alive; calls ``on_dead(ranks)`` once when one is not.

    Worker ranks of the multi-process server watch rank 0 with it: a worker blocked in the task broadcast of a rank 0
    that stopped (without closing its sockets) would otherwise wait forever, like the reference's workers in
    ``MPI_Bcast``.  The default action logs and leaves the process with exit code 3 -- between steps from the point of
    view of the device, because the worker is idle in a host-side wait when this fires."""

    def __init__(self, heartbeat: Heartbeat, ranks: List[int], on_dead=None, period: float = 0.5):
        self.hb, self.ranks, self.period = heartbeat, list(ranks), period
        self.on_dead = on_dead or self._exit
        self.fired = False
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    @staticmethod
    def _exit(ranks):
        import logging
        import os
        logging.getLogger("jittorinfer_b200.health").error("rank(s) %s stopped responding: leaving", ranks)
        os._exit(3)

    def start(self) -> "Watchdog":
        def loop():
            while not self._stop.wait(self.period):
                gone = self.hb.dead(self.ranks)
                if gone:
                    self.fired = True
                    self.on_dead(gone)
                    return
        self._thread = threading.Thread(target=loop, name="watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.period + 1)
