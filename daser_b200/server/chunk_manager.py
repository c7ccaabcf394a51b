"""FIFO ring allocator over the slots of the store file.

Capability parity: ``daser/server/chunk_manager.py:18-290`` — ``alloc`` with
wrap (skip run + head back to 0), ``evict_oldest``, ``free_slots``, ``head`` /
``tail``, ``save`` / ``load`` of ``{"head", "tail", "index", "doc_registry"}``,
eviction notifications to the ``DocRegistry``.

Design differences (each is a defect of the reference that callers can hit):

* Occupancy is an explicit ``used`` counter, so ``head == tail`` needs no
  "is the store empty" guess (``chunk_manager.py:74-85``); that guess breaks
  once explicit evictions can empty the index while slots are still held.
* Eviction listeners: whoever owns a retrieval index registers a callback and
  every eviction path (FIFO, wrap, explicit, abort) invalidates the index
  before the slots are reused; the reference never removes ring-evicted
  chunks from its index and serves stale hits.
* ``alloc`` checks for an existing key *before* mutating the ring and is
  idempotent for an uncommitted reservation of the same size
  (``get_num_new_matched_tokens`` may be called repeatedly by the engine).
* ``abort`` releases a reservation whose request died; if it was the newest
  allocation the head is rolled back.
* A ``cont`` slot at the tail is an invariant violation and raises.
* Snapshots are written atomically (tmp + fsync + rename) and carry the
  reservation state so a restart never publishes half-written chunks.
"""

from __future__ import annotations

from typing import Callable, Optional

import msgpack

from daser_b200 import metrics
from daser_b200.logging import init_logger
from daser_b200.server.doc_registry import DocRegistry
from daser_b200.server.metadata_store import ChunkMeta, MetadataStore, atomic_write

logger = init_logger(__name__)

EvictionListener = Callable[[ChunkMeta], None]


class RingInvariantError(RuntimeError):
    """The slot map and head/tail disagree (corrupt snapshot or a bug)."""


class ChunkManager:
    def __init__(
        self,
        total_slots: int,
        metadata_store: MetadataStore,
        doc_registry: Optional[DocRegistry] = None,
    ) -> None:
        if metadata_store.total_slots != total_slots:
            raise ValueError("metadata store and ring disagree on total_slots")
        self._total = total_slots
        self._store = metadata_store
        self._docs = doc_registry
        self._head = 0
        self._tail = 0
        self._used = 0
        self._listeners: list[EvictionListener] = []

    # -- wiring -------------------------------------------------------------

    @property
    def doc_registry(self) -> Optional[DocRegistry]:
        return self._docs

    def set_doc_registry(self, doc_registry: DocRegistry) -> None:
        self._docs = doc_registry

    def add_eviction_listener(self, fn: EvictionListener) -> None:
        """``fn(meta)`` runs for every chunk that leaves the store, before removal."""
        self._listeners.append(fn)

    # -- state --------------------------------------------------------------

    @property
    def store(self) -> MetadataStore:
        return self._store

    @property
    def total_slots(self) -> int:
        return self._total

    @property
    def head(self) -> int:
        return self._head

    @property
    def tail(self) -> int:
        return self._tail

    @property
    def used_slots(self) -> int:
        return self._used

    @property
    def free_slots(self) -> int:
        return self._total - self._used

    # -- allocation -----------------------------------------------------------

    def alloc(
        self,
        chunk_key: str,
        num_slots: int,
        token_count: int,
        model_id: str,
        pos_offset: int,
        committed: bool = True,
    ) -> int:
        """Reserve ``num_slots`` contiguous slots; returns the first slot.

        ``committed=False`` marks the chunk as a reservation (the control plane
        uses this; direct callers keep the reference's semantics).
        """
        if num_slots <= 0:
            raise ValueError("num_slots must be positive")
        if num_slots > self._total:
            raise ValueError(f"num_slots={num_slots} exceeds total_slots={self._total}")
        existing = self._store.get(chunk_key)
        if existing is not None:
            if (
                not self._store.is_committed(chunk_key)
                and existing.num_slots == num_slots
                and existing.model_id == model_id
            ):
                return existing.start_slot
            raise ValueError(f"chunk_key already exists: {chunk_key}")

        room_at_end = self._total - self._head
        if room_at_end < num_slots:
            # The run must not straddle the end of the file: pad and wrap.
            while self.free_slots < room_at_end:
                self.evict_oldest()
            self._store.insert_skip(self._head, room_at_end)
            self._used += room_at_end
            self._head = 0
            metrics.inc("ring.wraps")
        while self.free_slots < num_slots:
            self.evict_oldest()

        start = self._head
        self._store.insert(
            ChunkMeta(chunk_key, start, num_slots, token_count, pos_offset, model_id),
            committed=committed,
        )
        self._used += num_slots
        self._head = (start + num_slots) % self._total
        metrics.inc("ring.allocs")
        return start

    def evict_oldest(self) -> None:
        """Drop the run at the tail (a chunk, a tombstone or wrap padding)."""
        if self._used == 0:
            raise RuntimeError("evict_oldest called on empty ring buffer")
        entry = self._store.get_slot_entry(self._tail)
        if entry.kind == "cont" or entry.num_slots <= 0:
            raise RingInvariantError(f"no run head at tail slot {self._tail}")
        if entry.kind == "chunk":
            self._drop(entry.chunk_key)  # type: ignore[arg-type]
            metrics.inc("ring.evictions")
        self._store.clear_run(self._tail)
        self._tail = (self._tail + entry.num_slots) % self._total
        self._used -= entry.num_slots
        if self._used < 0:
            raise RingInvariantError("ring occupancy went negative")

    def evict_chunk(self, chunk_key: str) -> bool:
        """Explicit eviction; slots are reclaimed when the tail reaches them."""
        if self._store.get(chunk_key) is None:
            return False
        self._drop(chunk_key)
        self._skip_dead_tail()
        return True

    def abort(self, chunk_key: str) -> bool:
        """Release an uncommitted reservation; committed chunks are left alone."""
        meta = self._store.get(chunk_key)
        if meta is None or self._store.is_committed(chunk_key):
            return False
        self._drop(chunk_key)
        if (meta.start_slot + meta.num_slots) % self._total == self._head:
            self._store.clear_run(meta.start_slot)
            self._head = meta.start_slot
            self._used -= meta.num_slots
        self._skip_dead_tail()
        metrics.inc("ring.aborts")
        return True

    def _drop(self, chunk_key: str) -> None:
        meta = self._store.get(chunk_key)
        if meta is None:
            return
        for fn in self._listeners:
            fn(meta)
        if self._docs is not None:
            for doc_id in list(meta.doc_ids):
                self._docs.mark_chunk_evicted(doc_id, chunk_key)
        self._store.remove(chunk_key)

    def _skip_dead_tail(self) -> None:
        while self._used > 0:
            entry = self._store.get_slot_entry(self._tail)
            if entry.kind != "skip":
                break
            self._store.clear_run(self._tail)
            self._tail = (self._tail + entry.num_slots) % self._total
            self._used -= entry.num_slots
        if self._used == 0:
            # Empty ring: restart at 0 so large runs fit without padding.
            self._head = self._tail = 0

    # -- persistence ------------------------------------------------------------

    def to_bytes(self) -> bytes:
        payload = {
            "head": self._head,
            "tail": self._tail,
            "index": self._store.to_bytes(),
            "doc_registry": self._docs.to_dict() if self._docs is not None else {},
            "ext": {"used": self._used, **self._store.ext_state()},
        }
        return msgpack.packb(payload, use_bin_type=True)

    def save(self, path: str) -> None:
        atomic_write(path, self.to_bytes())
        logger.info(
            "[CHUNK] state saved to %s (head=%d tail=%d chunks=%d)",
            path,
            self._head,
            self._tail,
            len(self._store),
        )

    def load(self, path: str, drop_uncommitted: bool = True) -> None:
        """Replace the state with a snapshot.

        Reservations that were never committed are dropped: their bytes may be
        half-written.  Raises on any inconsistency; the caller cold-starts.
        """
        with open(path, "rb") as f:
            payload = msgpack.unpackb(f.read(), raw=False)
        store = MetadataStore(self._total)
        store.from_bytes(payload["index"])
        if store.total_slots != self._total:
            raise RingInvariantError(
                f"snapshot has {store.total_slots} slots, ring has {self._total}"
            )
        ext = payload.get("ext") or {}
        store.load_ext_state(ext)
        head, tail = int(payload["head"]), int(payload["tail"])
        used = self._walk(store, head, tail, ext.get("used"))
        # Commit the new state only after validation.
        self._store.__dict__.update(store.__dict__)
        self._head, self._tail, self._used = head, tail, used
        if self._docs is not None:
            self._docs.load_dict(payload.get("doc_registry", {}) or {})
        if drop_uncommitted:
            for key in list(ext.get("uncommitted", [])):
                self.abort(key)
        logger.info(
            "[CHUNK] state loaded from %s (head=%d tail=%d chunks=%d)",
            path,
            self._head,
            self._tail,
            len(self._store),
        )

    def _walk(
        self, store: MetadataStore, head: int, tail: int, used_hint: Optional[int]
    ) -> int:
        """Validate that runs tile ``[tail, head)``; return the occupancy."""
        if not (0 <= head < self._total and 0 <= tail < self._total):
            raise RingInvariantError("head/tail outside the ring")
        if head == tail:
            full = used_hint == self._total if used_hint is not None else len(store) > 0
            if not full:
                return 0
        pos, used = tail, 0
        while True:
            entry = store.get_slot_entry(pos)
            if entry.kind == "cont" or entry.num_slots <= 0:
                raise RingInvariantError(f"no run head at slot {pos}")
            used += entry.num_slots
            if used > self._total:
                raise RingInvariantError("runs exceed the ring size")
            pos = (pos + entry.num_slots) % self._total
            if pos == head:
                return used
