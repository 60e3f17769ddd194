"""Rank heartbeat and failure detection on the host.

Neither the reference's own code nor its vendored engines detect a lost rank (they rely on NCCL time-outs, reference
``backend/backend_fsdp.py:111-115`` sets none).  Here every rank beats a counter in the rendezvous store every
``Config.heartbeat_interval_s`` seconds from a daemon thread; the same thread reads the peers' counters.  A peer whose
counter has not moved for ``heartbeat_timeout_s`` seconds, or that announced its departure with :meth:`leave`, is reported
by :meth:`check`, which the trainer calls between steps, *before* it launches kernels that would wait for that peer.  The
survivors therefore learn of a failure on the host; the bounded in-kernel waits (``Config.comm_timeout_s``) are the second
line of defence for a peer that dies inside a step.

Nothing here touches a GPU: a rank may only leave between steps, with none of its kernels or collectives in flight.
"""
from __future__ import annotations

import os
import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    """One or more peers left the job or stopped beating."""

    def __init__(self, lost: List[int], left: List[int]):
        self.lost, self.left = list(lost), list(left)
        parts = []
        if left:
            parts.append(f"ranks {left} left the job")
        if lost:
            parts.append(f"ranks {lost} stopped sending heartbeats")
        super().__init__("; ".join(parts) or "rank failure")


def _connect_store():
    """A store connection of our own (the default store's socket belongs to the thread that runs collectives)."""
    addr, port = os.environ.get("MASTER_ADDR"), os.environ.get("MASTER_PORT")
    if addr and port:
        try:
            return dist.TCPStore(addr, int(port), is_master=False, wait_for_workers=False)
        except Exception:
            pass
    try:
        return dist.distributed_c10d._get_default_store()
    except Exception:
        return None


class Heartbeat:
    def __init__(self, rank: Optional[int] = None, world: Optional[int] = None, interval_s: float = 0.5, timeout_s: float = 30.0,
                 store=None, prefix: str = "ats/hb"):
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.interval_s, self.timeout_s = max(float(interval_s), 0.01), float(timeout_s)
        self.store = store if store is not None else _connect_store()
        self.prefix = prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        self._last_value: Dict[int, int] = {}
        self._last_change: Dict[int, float] = {}
        self._left: List[int] = []
        self._lost: List[int] = []
        self.beats = 0

    # -- store access (counters are read with add(key, 0): never blocks, missing keys read as 0) -------------------
    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def _beat(self) -> None:
        self.store.add(self._key("beat", self.rank), 1)
        self.beats += 1

    def _scan(self) -> None:
        now = time.monotonic()
        left, lost = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.add(self._key("left", r), 0) > 0:
                left.append(r)
                continue
            v = self.store.add(self._key("beat", r), 0)
            if v != self._last_value.get(r):
                self._last_value[r] = v
                self._last_change[r] = now
            elif now - self._last_change.get(r, now) > self.timeout_s:
                lost.append(r)
            self._last_change.setdefault(r, now)
        with self._lock:
            self._left, self._lost = left, lost

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self._beat()
                self._scan()
            except Exception:
                # the store itself is gone (rank 0 hosts it): every peer is unreachable from here
                with self._lock:
                    self._lost = [r for r in range(self.world) if r != self.rank]
                return
            self._stop.wait(self.interval_s)

    # -- public ----------------------------------------------------------------------------------------------
    def start(self) -> "Heartbeat":
        if self.store is None or self.world <= 1 or self._thread is not None:
            return self
        self._thread = threading.Thread(target=self._run, name="ats-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        """Stops beating without announcing a departure (what a crashed or hung rank looks like to its peers)."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1.0)
            self._thread = None

    def leave(self) -> None:
        """Announce an orderly departure (call between steps, with no kernel or collective in flight) and stop beating."""
        if self.store is not None:
            try:
                self.store.add(self._key("left", self.rank), 1)
            except Exception:
                pass
        self.stop()

    def failed(self) -> bool:
        with self._lock:
            return bool(self._left or self._lost)

    def check(self) -> None:
        """Raise :class:`RankFailure` if a peer is gone.  Cheap: reads two lists the watchdog thread maintains."""
        with self._lock:
            left, lost = list(self._left), list(self._lost)
        if left or lost:
            raise RankFailure(lost, left)
