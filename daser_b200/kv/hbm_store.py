"""Memory tiers: hot chunks kept compressed in GPU memory (and warm ones in pinned host
memory), in front of the NVMe store.

No counterpart in the reference (its roadmap mentions tiered prefetch only).  Chunks are
kept in the on-disk slot format (fp8b16 images), so the restore kernel reads them exactly as
it reads a staging buffer and a hit costs no IO, no PCIe copy and no format conversion.

The arena is one device allocation of ``capacity_slots`` slots.  Chunks occupy contiguous
slot runs (the restore work list takes one base address per chunk); replacement is LRU with
first-fit placement: least-recently-used chunks are evicted until a large enough free run
exists.  Keys are content hashes, so an entry never goes stale.

The same class is the **host tier** when its arena is pinned host memory
(``HBMStore(..., device=torch.device("cpu"))``): pinned memory is addressable from the GPU, so
the restore kernel reads a warm chunk straight over PCIe, and a cold chunk is read from the
file directly into its reserved arena slots (``reserve``) with no staging copy.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch

from daser_b200 import metrics


class HBMStore:
    def __init__(self, slot_size: int, capacity_slots: int, device: Optional[torch.device] = None) -> None:
        if slot_size <= 0 or capacity_slots <= 0:
            raise ValueError("slot_size and capacity_slots must be positive")
        self.slot_size = slot_size
        self.capacity = capacity_slots
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if self.device.type == "cpu":
            self.arena = torch.empty(slot_size * capacity_slots, dtype=torch.uint8)
            if torch.cuda.is_available():
                self.arena = self.arena.pin_memory()
        else:
            self.arena = torch.empty(slot_size * capacity_slots, dtype=torch.uint8, device=self.device)
        self.kind = "host" if self.device.type == "cpu" else "hbm"
        self._protected: set[str] = set()
        self._chunks: "OrderedDict[str, tuple[int, int]]" = OrderedDict()  # key -> (first slot, n)
        self._free: list[tuple[int, int]] = [(0, capacity_slots)]  # sorted (first slot, n) runs

    # -- queries ----------------------------------------------------------------------------
    def __contains__(self, key: str) -> bool:
        return key in self._chunks

    def __len__(self) -> int:
        return len(self._chunks)

    @property
    def used_slots(self) -> int:
        return sum(n for _, n in self._chunks.values())

    def lookup(self, key: str, need_slots: int = 0) -> Optional[int]:
        """Device address of the chunk's first slot image, or None.

        ``need_slots`` is how many slots from the start of the chunk the caller is going to read;
        an entry that holds fewer is not a hit (and is dropped, so that the whole chunk can be
        cached in its place)."""
        hit = self._chunks.get(key)
        if hit is not None and hit[1] < need_slots:
            self.evict(key)
            hit = None
        if hit is None:
            metrics.inc(f"{self.kind}.misses")
            return None
        self._chunks.move_to_end(key)
        self._protected.add(key)
        metrics.inc(f"{self.kind}.hits")
        return self.arena.data_ptr() + hit[0] * self.slot_size

    def end_step(self) -> None:
        """Entries looked up or reserved since the last call may be evicted again."""
        self._protected.clear()
        metrics.set_gauge(f"{self.kind}.used_slots", self.used_slots)
        metrics.set_gauge(f"{self.kind}.capacity_slots", self.capacity)

    # -- placement -----------------------------------------------------------------------------
    def _take(self, n: int) -> Optional[int]:
        for i, (first, run) in enumerate(self._free):
            if run >= n:
                if run == n:
                    self._free.pop(i)
                else:
                    self._free[i] = (first + n, run - n)
                return first
        return None

    def _release(self, first: int, n: int) -> None:
        self._free.append((first, n))
        self._free.sort()
        merged: list[tuple[int, int]] = []
        for f, r in self._free:
            if merged and merged[-1][0] + merged[-1][1] == f:
                merged[-1] = (merged[-1][0], merged[-1][1] + r)
            else:
                merged.append((f, r))
        self._free = merged

    def evict(self, key: str) -> bool:
        hit = self._chunks.pop(key, None)
        if hit is None:
            return False
        self._release(*hit)
        self._protected.discard(key)
        metrics.inc(f"{self.kind}.evictions")
        return True

    def clear(self) -> int:
        """Forget every entry (the arena stays allocated); returns how many there were."""
        n = len(self._chunks)
        self._chunks.clear()
        self._protected.clear()
        self._free = [(0, self.capacity)]
        if n:
            metrics.inc(f"{self.kind}.evictions", n)
        return n

    def reserve(self, key: str, nbytes: int) -> Optional[int]:
        """Claim room for ``key`` and return the arena byte offset to fill (None if it cannot fit
        without evicting an entry that the current step still reads)."""
        if nbytes % self.slot_size:
            raise ValueError("chunk size is not a whole number of slots")
        n = nbytes // self.slot_size
        if key in self._chunks:
            if self._chunks[key][1] >= n:
                self._chunks.move_to_end(key)
                self._protected.add(key)
                return self._chunks[key][0] * self.slot_size
            if key in self._protected:
                return None  # a shorter entry that this step still reads
            self.evict(key)
        if n > self.capacity:
            return None
        first = self._take(n)
        while first is None:
            victim = next((k for k in self._chunks if k not in self._protected), None)
            if victim is None:
                return None
            self.evict(victim)
            first = self._take(n)
        self._chunks[key] = (first, n)
        self._protected.add(key)
        return first * self.slot_size

    def admit(self, key: str, src: torch.Tensor, src_offset: int, nbytes: int) -> bool:
        """Copy ``nbytes`` of slot images from ``src`` (pinned host or device uint8 tensor).

        The copy is enqueued on the current stream.  Returns False when the chunk is larger
        than the arena; an existing entry is only touched.
        """
        if key in self._chunks:
            self._chunks.move_to_end(key)
            self._protected.add(key)  # like every other touch: stays until the step ends
            return True
        off = self.reserve(key, nbytes)
        if off is None:
            return False
        self.arena[off : off + nbytes].copy_(src[src_offset : src_offset + nbytes], non_blocking=True)
        metrics.inc(f"{self.kind}.admitted_bytes", nbytes)
        return True

    def stats(self) -> dict[str, float]:
        return {"chunks": len(self._chunks), "used_slots": self.used_slots, "capacity_slots": self.capacity}
