"""Peer liveness for the tensor-parallel group: leave notices, heartbeats, host-side checks.

The fused tensor-parallel kernels wait on flags that other ranks set.  Those waits are
bounded (they give up after a time budget and report through a status word), but a step that
starts after a peer is gone still costs that budget on every sync point.  So liveness is
settled on the host, between steps, before anything is launched:

* a rank that stops in an orderly way calls :meth:`PeerMonitor.leave` between steps; it bumps
  a counter in the group's key-value store, and the other ranks see it at their next
  :meth:`PeerMonitor.check` (one store round trip);
* a rank that crashed leaves nothing behind, so every rank also runs a heartbeat thread that
  writes a timestamp under its own key and reads the others'; a peer whose heartbeat is older
  than ``timeout_s`` is reported by the next ``check``;
* a store that no longer answers (it lives in rank 0's process) counts as rank 0 lost.

``check`` raises :class:`PeerLost` with the ranks it found missing.  The engine treats that as
fatal for the current group: requests in flight are failed, the group is torn down with no
kernels in flight, and the surviving ranks can be started again as a smaller group (weights are
re-sharded from the checkpoint; the KV store on disk is tensor-parallel agnostic, so every
stored chunk remains usable at the new degree).

The reference is a single process with no peers and no liveness checks of any kind; its only
failure handling is the socket timeout and retry of ``daser/connector/ipc_client.py:76,103-115``.
Works with any ``torch.distributed`` store, so the logic is tested with CPU processes.
"""

from __future__ import annotations

import threading
import time
from typing import Any, Optional, Sequence

from daser_b200 import metrics
from daser_b200.logging import init_logger

logger = init_logger(__name__)


class PeerLost(RuntimeError):
    def __init__(self, ranks: Sequence[int], why: str) -> None:
        super().__init__(f"tensor-parallel peer(s) {sorted(ranks)} lost: {why}")
        self.ranks = sorted(ranks)
        self.why = why


class PeerMonitor:
    """Liveness of ``world`` ranks over a ``torch.distributed`` store.

    ``store`` is any object with ``set(key, bytes)``, ``get(key)``, ``add(key, int)`` and
    ``check([keys])`` (``TCPStore``, ``FileStore``, ``HashStore``, ``PrefixStore``).
    """

    def __init__(self, store: Any, rank: int, world: int, *, timeout_s: float = 5.0,
                 interval_s: float = 0.5, prefix: str = "daser/health", start: bool = True) -> None:
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.interval_s = timeout_s, interval_s
        self._prefix = prefix
        self._lost: dict[int, str] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_seen = {r: time.monotonic() for r in range(world)}
        self._last_value: dict[int, bytes] = {}
        self._left = False
        self._beat()
        if start and world > 1:
            self._thread = threading.Thread(target=self._run, name="daser-health", daemon=True)
            self._thread.start()

    # -- keys ---------------------------------------------------------------------------------
    def _key(self, what: str, rank: Optional[int] = None) -> str:
        return f"{self._prefix}/{what}" if rank is None else f"{self._prefix}/{what}/{rank}"

    def _beat(self) -> None:
        self.store.set(self._key("hb", self.rank), repr(time.time()).encode())

    # -- background heartbeat --------------------------------------------------------------------
    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
                self.poll()
            except Exception as exc:  # the store went away with its host process
                self._mark(0, f"store unreachable ({type(exc).__name__})")
                return

    def poll(self) -> None:
        """One pass over the peers' heartbeats (the background thread calls this)."""
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key("hb", r)
            if not self.store.check([key]):
                value = b""
            else:
                value = bytes(self.store.get(key))
            if value and value != self._last_value.get(r):
                self._last_value[r] = value
                self._last_seen[r] = now
            elif now - self._last_seen[r] > self.timeout_s:
                self._mark(r, f"no heartbeat for {now - self._last_seen[r]:.1f} s")

    def _mark(self, rank: int, why: str) -> None:
        with self._lock:
            if rank not in self._lost:
                self._lost[rank] = why
                metrics.inc("tp.peer_lost")
                logger.error("[TP] rank %d: peer %d lost: %s", self.rank, rank, why)

    # -- what the engine calls between steps ---------------------------------------------------------
    def check(self) -> None:
        """Raise :class:`PeerLost` if any peer left or stopped beating.  One store round trip."""
        if self.world <= 1:
            return
        try:
            departed = int(self.store.add(self._key("left_count"), 0))
        except Exception as exc:
            self._mark(0, f"store unreachable ({type(exc).__name__})")
            departed = 0
        if departed:
            for r in range(self.world):
                if r != self.rank and r not in self._lost and self.store.check([self._key("left", r)]):
                    self._mark(r, "left the group")
        with self._lock:
            lost = dict(self._lost)
        if lost:
            raise PeerLost(list(lost), "; ".join(f"{r}: {w}" for r, w in sorted(lost.items())))

    def lost(self) -> list[int]:
        with self._lock:
            return sorted(self._lost)

    def leave(self) -> None:
        """Orderly exit: call between steps, with none of this rank's kernels in flight."""
        if self._left:
            return
        self._left = True
        self.close()
        try:
            self.store.set(self._key("left", self.rank), b"1")
            self.store.add(self._key("left_count"), 1)
        except Exception:  # nobody left to tell
            pass

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2 * self.interval_s + 1)
        self._thread = None
