"""Host-side mailboxes in shared memory: how the ranks of one box pass small control messages.

Every engine step of a tensor-parallel engine starts with the same few hundred bytes on every
rank: which chunks were found, where they go, who reads them.  Sent as a pickled object through
a gloo broadcast that costs two collectives and a few hundred microseconds inside every time to
first token.  All ranks of this engine live on one machine, so the message goes through a
POSIX shared-memory segment instead: each rank owns a small ring of slots; a writer fills the
next slot and then stamps it with the message's number; readers wait (bounded) for the number
they expect and copy the payload out.  A publish and its reads take about ten microseconds.

The reference has no multi-rank engine and therefore nothing like it.
"""

from __future__ import annotations

import mmap
import os
import pickle
import struct
import time
from typing import Any, Optional

_HDR = struct.Struct("<QQ")  # message number, payload length (the slot header)
_U64 = struct.Struct("<Q")


class MailboxTimeout(TimeoutError):
    """A peer did not publish in time (it left, crashed, or runs far behind)."""


class HostMailbox:
    RING = 4  # messages of one writer that may be outstanding before a reader is overrun

    def __init__(self, path: str, rank: int, world: int, slot_bytes: int = 1 << 18, create: bool = False) -> None:
        self.path, self.rank, self.world, self.slot_bytes = path, rank, world, slot_bytes
        size = world * self.RING * slot_bytes
        flags = os.O_RDWR | (os.O_CREAT | os.O_EXCL if create else 0)
        fd = os.open(path, flags, 0o600)
        try:
            if create:
                os.ftruncate(fd, size)
            self._mm = mmap.mmap(fd, size)
        finally:
            os.close(fd)
        self._created = create
        self._seen = [0] * world  # number of the last message consumed from each rank
        self._sent = 0  # number of this rank's last message

    @staticmethod
    def default_path(tag: str) -> str:
        base = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
        return os.path.join(base, f"daser_mailbox_{tag}")

    def _base(self, rank: int, number: int) -> int:
        return (rank * self.RING + number % self.RING) * self.slot_bytes

    # -- writer -----------------------------------------------------------------------------
    def publish(self, obj: Any) -> None:
        """Append ``obj`` to this rank's messages (message n lives in sub-slot n mod RING)."""
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        if len(data) > self.slot_bytes - _HDR.size:
            raise ValueError(f"message of {len(data)} bytes exceeds the mailbox slot")
        self._sent += 1
        base = self._base(self.rank, self._sent)
        mm = self._mm
        _U64.pack_into(mm, base, 0)  # being written
        mm[base + _HDR.size : base + _HDR.size + len(data)] = data
        _U64.pack_into(mm, base + 8, len(data))
        _U64.pack_into(mm, base, self._sent)  # last, as a store of its own: the number publishes the rest

    # -- reader -----------------------------------------------------------------------------
    def receive(self, src: int, timeout_s: float = 30.0, on_wait=None) -> Any:
        """The next message of rank ``src`` that this rank has not consumed yet.

        Messages are consumed in order.  A writer that gets RING messages ahead of a reader has
        overwritten what the reader still wanted; that is reported, not papered over.
        ``on_wait`` is called now and then while waiting (peer liveness checks) and may raise."""
        want = self._seen[src] + 1
        base = self._base(src, want)
        mm = self._mm
        t0 = time.perf_counter()
        spins = 0
        slow = False
        while True:
            (seq,) = _U64.unpack_from(mm, base)
            if seq == want:
                (n,) = _U64.unpack_from(mm, base + 8)
                data = bytes(mm[base + _HDR.size : base + _HDR.size + n])
                (seq2,) = _U64.unpack_from(mm, base)
                if seq2 == seq:
                    self._seen[src] = seq
                    return pickle.loads(data)
                seq = seq2
            if seq > want:
                raise RuntimeError(f"mailbox overrun: rank {src} is at message {seq}, message {want} was lost")
            spins += 1
            if spins & 0x3FF and not slow:
                continue  # the first milliseconds: a tight poll (a step's plan arrives within microseconds)
            waited = time.perf_counter() - t0
            if waited > timeout_s:
                raise MailboxTimeout(f"rank {src} published nothing for {timeout_s:.0f} s")
            if on_wait is not None and (not slow or spins & 0x3F == 0):
                on_wait()
            if waited > 0.002:
                # nothing came at once: back off (an idle service's follower costs next to nothing,
                # and the first request after the pause pays at most the last sleep)
                slow = True
                time.sleep(0.005 if waited > 1.0 else 0.001 if waited > 0.05 else 0.0001)

    def broadcast(self, obj: Any, src: int = 0, timeout_s: float = 30.0, on_wait=None) -> Any:
        """``obj`` of rank ``src`` on every rank (the others pass anything)."""
        if self.rank == src:
            self.publish(obj)
            return obj
        return self.receive(src, timeout_s, on_wait)

    def gather(self, obj: Any, timeout_s: float = 30.0, on_wait=None) -> list[Any]:
        """Every rank's ``obj``, in rank order, on every rank."""
        self.publish(obj)
        return [obj if r == self.rank else self.receive(r, timeout_s, on_wait) for r in range(self.world)]

    def close(self) -> None:
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass
        if self._created:
            try:
                os.unlink(self.path)
            except OSError:
                pass


def open_mailbox(rank: int, world: int, exchange, slot_bytes: int = 1 << 18) -> Optional[HostMailbox]:
    """Create the segment on rank 0, tell the others its path through ``exchange`` (a broadcast
    callable ``exchange(obj) -> obj of rank 0``), open it there.  One barrier-like call at start-up."""
    path = None
    box = None
    if rank == 0:
        path = HostMailbox.default_path(f"{os.getpid()}_{time.time_ns() & 0xFFFFFF:x}")
        box = HostMailbox(path, rank, world, slot_bytes, create=True)
    path = exchange(path)
    if rank != 0:
        box = HostMailbox(path, rank, world, slot_bytes, create=False)
    return box
