"""Exact longest-prefix index.

Capability parity: ``daser/retrieval/prefix.py:33-90`` — keys are the XXH3-128
digest of a block-aligned token prefix; ``lookup`` returns at most one chunk,
the longest stored prefix of the query whose ``model_id`` matches.

The reference re-hashes every candidate prefix from scratch (quadratic in the
prompt length).  Here all block-aligned prefix digests come from one streaming
pass (:func:`daser_b200.hashing.prefix_digests`), then the dict is probed from
the longest prefix down.  When the native index is built (``server/csrc/token_index.cc``) the
whole query is one call: the digests are computed and probed in C++ against a table keyed by
(model, digest), and only the winning chunk's handle comes back.
"""

from __future__ import annotations

import xxhash

from daser_b200.hashing import prefix_digests
from daser_b200.retrieval.base import RetrievalIndex
from daser_b200.server import native_index
from daser_b200.server.metadata_store import ChunkMeta


def _is_digest(key: str) -> bool:
    """Only keys that are XXH3-128 hex digests can ever equal the digest of a token prefix."""
    if len(key) != 32:
        return False
    try:
        bytes.fromhex(key)
    except ValueError:
        return False
    return True


def model_tag(model_id: str) -> int:
    """64-bit tag that keys a model's entries in the native table."""
    return xxhash.xxh3_64(model_id.encode()).intdigest()


class PrefixHashIndex(RetrievalIndex):
    def __init__(self, block_tokens: int = 16, native: bool | None = None) -> None:
        if block_tokens <= 0:
            raise ValueError("block_tokens must be positive")
        self._block_tokens = block_tokens
        self._by_key: dict[str, ChunkMeta] = {}
        use_native = native_index.available() if native is None else (native and native_index.available())
        self._table = native_index.DigestTable() if use_native else None
        self._handles: dict[int, ChunkMeta] = {}
        self._handle_of: dict[str, int] = {}
        self._next_handle = 0

    @property
    def native(self) -> bool:
        return self._table is not None

    def _table_insert(self, meta: ChunkMeta) -> None:
        if self._table is None or not _is_digest(meta.chunk_key):
            return
        self._table_remove(meta.chunk_key)
        handle = self._next_handle
        self._next_handle += 1
        self._handles[handle] = meta
        self._handle_of[meta.chunk_key] = handle
        self._table.put(model_tag(meta.model_id), meta.chunk_key, handle)

    def _table_remove(self, chunk_key: str) -> None:
        if self._table is None:
            return
        handle = self._handle_of.pop(chunk_key, None)
        if handle is not None:
            meta = self._handles.pop(handle)
            self._table.delete(model_tag(meta.model_id), chunk_key)

    def lookup_sync(self, tokens: list[int], model_id: str) -> list[ChunkMeta]:
        if not self._by_key:
            return []
        if self._table is not None:
            handle, _ = self._table.longest_prefix(model_tag(model_id), tokens, self._block_tokens)
            return [self._handles[handle]] if handle >= 0 else []
        for digest in reversed(prefix_digests(tokens, self._block_tokens)):
            meta = self._by_key.get(digest)
            if meta is not None and meta.model_id == model_id:
                return [meta]
        return []

    async def lookup(self, tokens: list[int], model_id: str) -> list[ChunkMeta]:
        return self.lookup_sync(tokens, model_id)

    def get(self, chunk_key: str) -> ChunkMeta | None:
        return self._by_key.get(chunk_key)

    async def insert(self, meta: ChunkMeta) -> None:
        self._by_key[meta.chunk_key] = meta
        self._table_insert(meta)

    async def remove(self, chunk_key: str) -> None:
        self._by_key.pop(chunk_key, None)
        self._table_remove(chunk_key)

    def discard(self, chunk_key: str) -> None:
        self._by_key.pop(chunk_key, None)
        self._table_remove(chunk_key)

    def __len__(self) -> int:
        return len(self._by_key)
