"""HBM tier: hot chunks kept compressed in GPU memory, in front of the NVMe store.

No counterpart in the reference (its roadmap mentions tiered prefetch only).  Chunks are
kept in the on-disk slot format (fp8b16 images), so the restore kernel reads them exactly as
it reads a staging buffer and a hit costs no IO, no PCIe copy and no format conversion.

The arena is one device allocation of ``capacity_slots`` slots.  Chunks occupy contiguous
slot runs (the restore work list takes one base address per chunk); replacement is LRU with
first-fit placement: least-recently-used chunks are evicted until a large enough free run
exists.  Keys are content hashes, so an entry never goes stale.
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
        self.arena = torch.empty(slot_size * capacity_slots, dtype=torch.uint8, device=self.device)
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

    def lookup(self, key: str) -> Optional[int]:
        """Device address of the chunk's first slot image, or None."""
        hit = self._chunks.get(key)
        if hit is None:
            metrics.inc("hbm.misses")
            return None
        self._chunks.move_to_end(key)
        metrics.inc("hbm.hits")
        return self.arena.data_ptr() + hit[0] * self.slot_size

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
        metrics.inc("hbm.evictions")
        return True

    def admit(self, key: str, src: torch.Tensor, src_offset: int, nbytes: int) -> bool:
        """Copy ``nbytes`` of slot images from ``src`` (pinned host or device uint8 tensor).

        The copy is enqueued on the current stream.  Returns False when the chunk is larger
        than the arena; an existing entry is only touched.
        """
        if key in self._chunks:
            self._chunks.move_to_end(key)
            return True
        if nbytes % self.slot_size:
            raise ValueError("chunk size is not a whole number of slots")
        n = nbytes // self.slot_size
        if n > self.capacity:
            return False
        first = self._take(n)
        while first is None:
            if not self._chunks:
                return False
            victim = next(iter(self._chunks))
            self.evict(victim)
            first = self._take(n)
        dst = self.arena[first * self.slot_size : first * self.slot_size + nbytes]
        dst.copy_(src[src_offset : src_offset + nbytes], non_blocking=True)
        self._chunks[key] = (first, n)
        metrics.inc("hbm.admitted_bytes", nbytes)
        return True

    def stats(self) -> dict[str, float]:
        return {"chunks": len(self._chunks), "used_slots": self.used_slots, "capacity_slots": self.capacity}
