"""Exact longest-prefix index.

Capability parity: ``daser/retrieval/prefix.py:33-90`` — keys are the XXH3-128
digest of a block-aligned token prefix; ``lookup`` returns at most one chunk,
the longest stored prefix of the query whose ``model_id`` matches.

The reference re-hashes every candidate prefix from scratch (quadratic in the
prompt length).  Here all block-aligned prefix digests come from one streaming
pass (:func:`daser_b200.hashing.prefix_digests`), then the dict is probed from
the longest prefix down.
"""

from __future__ import annotations

from daser_b200.hashing import prefix_digests
from daser_b200.retrieval.base import RetrievalIndex
from daser_b200.server.metadata_store import ChunkMeta


class PrefixHashIndex(RetrievalIndex):
    def __init__(self, block_tokens: int = 16) -> None:
        if block_tokens <= 0:
            raise ValueError("block_tokens must be positive")
        self._block_tokens = block_tokens
        self._by_key: dict[str, ChunkMeta] = {}

    def lookup_sync(self, tokens: list[int], model_id: str) -> list[ChunkMeta]:
        if not self._by_key:
            return []
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

    async def remove(self, chunk_key: str) -> None:
        self._by_key.pop(chunk_key, None)

    def discard(self, chunk_key: str) -> None:
        self._by_key.pop(chunk_key, None)

    def __len__(self) -> int:
        return len(self._by_key)
