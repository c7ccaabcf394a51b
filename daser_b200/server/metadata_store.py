"""Chunk metadata and the slot map of the ring.

Capability parity: ``daser/server/metadata_store.py:17-240`` (``ChunkMeta``,
``SlotEntry``, ``MetadataStore`` with insert / insert_skip / remove / get /
get_slot_entry / iter_chunks / save / load and the msgpack payload
``{"total_slots", "chunk_index", "slot_map"}``).

Design differences:

* The slot map is stored as *runs* (a dict keyed by the first slot of each
  chunk or skip run) instead of one Python object per slot; a store of a few
  million slots therefore costs memory proportional to the number of chunks.
  :meth:`get_slot_entry` still answers for every slot id, and the snapshot is
  expanded to the reference's one-entry-per-slot list so either implementation
  can read the other's file.
* :meth:`remove` turns the chunk's run into a skip run (a tombstone) instead
  of leaving a dangling ``kind="chunk"`` head, so an explicit eviction followed
  by ring reclamation of the same slots cannot raise ``KeyError``
  (``daser/server/chunk_manager.py:164-173`` vs ``ipc_server.py:326``).
* Reservation state (``committed``) and the optional payload checksum live in
  a side table so that ``chunk_index`` entries keep exactly the reference's
  eight fields.
"""

from __future__ import annotations

import os
import time
from dataclasses import asdict, dataclass, field
from typing import Iterator, Literal, Optional

import msgpack

from daser_b200.logging import init_logger

logger = init_logger(__name__)

SlotKind = Literal["chunk", "skip", "cont"]


@dataclass
class ChunkMeta:
    """One cached KV chunk: ``num_slots`` contiguous slots from ``start_slot``."""

    chunk_key: str
    start_slot: int
    num_slots: int
    token_count: int
    pos_offset: int
    model_id: str
    created_at: float = 0.0
    doc_ids: list[str] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.created_at == 0.0:
            self.created_at = time.time()


@dataclass
class SlotEntry:
    """Per-slot view: ``chunk``/``skip`` on the first slot of a run, else ``cont``."""

    kind: SlotKind
    chunk_key: Optional[str] = None
    num_slots: int = 0


_CONT = SlotEntry(kind="cont")


class MetadataStore:
    """``chunk_key -> ChunkMeta`` plus the run map used for ring traversal."""

    def __init__(self, total_slots: int) -> None:
        if total_slots <= 0:
            raise ValueError("total_slots must be positive")
        self._total_slots = total_slots
        self._chunks: dict[str, ChunkMeta] = {}
        self._runs: dict[int, SlotEntry] = {}
        self._uncommitted: set[str] = set()
        self._checksums: dict[str, int] = {}
        self._anchors: dict[str, str] = {}  # chunk_key -> digest of its first block (chunk-offset scan)

    # -- mutation ---------------------------------------------------------

    def _check_range(self, start: int, n: int) -> None:
        if n <= 0 or start < 0 or start + n > self._total_slots:
            raise ValueError(
                f"slot run [{start}, {start + n}) outside [0, {self._total_slots})"
            )

    def _clear_heads(self, start: int, n: int) -> None:
        """Drop run heads strictly inside (start, start+n): they become ``cont``."""
        if len(self._runs) < n:
            for s in [s for s in self._runs if start < s < start + n]:
                del self._runs[s]
        else:
            for s in range(start + 1, start + n):
                self._runs.pop(s, None)

    def insert(self, meta: ChunkMeta, committed: bool = True) -> None:
        if meta.chunk_key in self._chunks:
            raise ValueError(f"chunk_key already exists: {meta.chunk_key}")
        self._check_range(meta.start_slot, meta.num_slots)
        self._chunks[meta.chunk_key] = meta
        self._runs[meta.start_slot] = SlotEntry(
            "chunk", meta.chunk_key, meta.num_slots
        )
        self._clear_heads(meta.start_slot, meta.num_slots)
        if not committed:
            self._uncommitted.add(meta.chunk_key)

    def insert_skip(self, start_slot: int, num_slots: int) -> None:
        self._check_range(start_slot, num_slots)
        self._runs[start_slot] = SlotEntry("skip", None, num_slots)
        self._clear_heads(start_slot, num_slots)

    def remove(self, chunk_key: str) -> None:
        """Forget ``chunk_key``; its slots become a skip run until reclaimed."""
        meta = self._chunks.pop(chunk_key, None)
        if meta is None:
            raise KeyError(f"chunk_key not found: {chunk_key}")
        head = self._runs.get(meta.start_slot)
        if head is not None and head.kind == "chunk" and head.chunk_key == chunk_key:
            self._runs[meta.start_slot] = SlotEntry("skip", None, meta.num_slots)
        self._uncommitted.discard(chunk_key)
        self._checksums.pop(chunk_key, None)
        self._anchors.pop(chunk_key, None)

    def clear_run(self, start_slot: int) -> None:
        """Erase the run head at ``start_slot`` (the ring reclaimed these slots)."""
        self._runs.pop(start_slot, None)

    def mark_committed(self, chunk_key: str, checksum: Optional[int] = None, anchor: Optional[str] = None) -> None:
        if chunk_key not in self._chunks:
            raise KeyError(f"chunk_key not found: {chunk_key}")
        self._uncommitted.discard(chunk_key)
        if checksum is not None:
            self._checksums[chunk_key] = int(checksum)
        if anchor:
            self._anchors[chunk_key] = str(anchor)

    # -- query ------------------------------------------------------------

    @property
    def total_slots(self) -> int:
        return self._total_slots

    def get(self, chunk_key: str) -> Optional[ChunkMeta]:
        return self._chunks.get(chunk_key)

    def is_committed(self, chunk_key: str) -> bool:
        return chunk_key in self._chunks and chunk_key not in self._uncommitted

    def checksum(self, chunk_key: str) -> Optional[int]:
        return self._checksums.get(chunk_key)

    def anchor(self, chunk_key: str) -> Optional[str]:
        """Digest of the chunk's first block, as given at commit (kept across restarts)."""
        return self._anchors.get(chunk_key)

    def get_slot_entry(self, slot_id: int) -> SlotEntry:
        if not 0 <= slot_id < self._total_slots:
            raise IndexError(f"slot {slot_id} outside [0, {self._total_slots})")
        return self._runs.get(slot_id, _CONT)

    def runs_in(self, start: int, count: int) -> list[tuple[int, SlotEntry]]:
        """Run heads whose first slot lies in ``[start, start+count)``, ascending."""
        if len(self._runs) < count:
            hits = [(s, e) for s, e in self._runs.items() if start <= s < start + count]
            hits.sort(key=lambda kv: kv[0])
            return hits
        return [
            (s, self._runs[s]) for s in range(start, start + count) if s in self._runs
        ]

    def __len__(self) -> int:
        return len(self._chunks)

    def iter_chunks(self) -> Iterator[ChunkMeta]:
        return iter(list(self._chunks.values()))

    # -- persistence --------------------------------------------------------

    def to_bytes(self) -> bytes:
        slot_map = [
            {"kind": "cont", "chunk_key": None, "num_slots": 0}
        ] * self._total_slots
        slot_map = list(slot_map)
        for start, entry in self._runs.items():
            slot_map[start] = {
                "kind": entry.kind,
                "chunk_key": entry.chunk_key,
                "num_slots": entry.num_slots,
            }
        payload = {
            "total_slots": self._total_slots,
            "chunk_index": {k: asdict(v) for k, v in self._chunks.items()},
            "slot_map": slot_map,
        }
        return msgpack.packb(payload, use_bin_type=True)

    def from_bytes(self, raw: bytes) -> None:
        payload = msgpack.unpackb(raw, raw=False)
        total = int(payload["total_slots"])
        chunks = {k: ChunkMeta(**v) for k, v in payload["chunk_index"].items()}
        runs: dict[int, SlotEntry] = {}
        for slot, e in enumerate(payload["slot_map"]):
            if e["kind"] != "cont":
                runs[slot] = SlotEntry(e["kind"], e.get("chunk_key"), e["num_slots"])
        # A head left behind by the reference's non-tombstoning remove()
        # names a key that no longer exists: demote it to a skip run.
        for slot, e in runs.items():
            if e.kind == "chunk" and e.chunk_key not in chunks:
                runs[slot] = SlotEntry("skip", None, e.num_slots)
        self._total_slots, self._chunks, self._runs = total, chunks, runs
        self._uncommitted = set()
        self._checksums = {}
        self._anchors = {}

    def ext_state(self) -> dict:
        return {
            "uncommitted": sorted(self._uncommitted),
            "checksums": dict(self._checksums),
            "anchors": dict(self._anchors),
        }

    def load_ext_state(self, ext: dict) -> None:
        self._uncommitted = {k for k in ext.get("uncommitted", []) if k in self._chunks}
        self._checksums = {
            k: int(v) for k, v in ext.get("checksums", {}).items() if k in self._chunks
        }
        self._anchors = {k: str(v) for k, v in ext.get("anchors", {}).items() if k in self._chunks}

    def save(self, path: str) -> None:
        atomic_write(path, self.to_bytes())
        logger.info("[INDEX] saved %d chunks to %s", len(self._chunks), path)

    def load(self, path: str) -> None:
        with open(path, "rb") as f:
            self.from_bytes(f.read())
        logger.info("[INDEX] loaded %d chunks from %s", len(self._chunks), path)


def atomic_write(path: str, data: bytes) -> None:
    """Write ``data`` so a crash leaves either the old or the new file.

    The reference writes snapshots in place with no fsync
    (``daser/server/chunk_manager.py:209-210``).
    """
    tmp = f"{path}.tmp.{os.getpid()}"
    fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
    try:
        view = memoryview(data)
        while view:
            n = os.write(fd, view)
            view = view[n:]
        os.fsync(fd)
    finally:
        os.close(fd)
    os.replace(tmp, path)
    dfd = os.open(os.path.dirname(os.path.abspath(path)), os.O_RDONLY)
    try:
        os.fsync(dfd)
    finally:
        os.close(dfd)
