"""Retrieval index plug-in point.

Capability parity: ``daser/retrieval/base.py:10-48`` — async ``lookup`` (best
match first), ``insert``, ``remove``.  Added: :meth:`discard`, a synchronous
removal that ring eviction calls from inside the allocator so the index can
never name slots that were handed to another chunk.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

from daser_b200.server.metadata_store import ChunkMeta


class RetrievalIndex(ABC):
    @abstractmethod
    async def lookup(self, tokens: list[int], model_id: str) -> list[ChunkMeta]:
        """Chunks usable for ``tokens``, most useful first; empty on a miss."""

    @abstractmethod
    async def insert(self, meta: ChunkMeta) -> None:
        """Make ``meta`` visible to lookups (second phase of the commit)."""

    @abstractmethod
    async def remove(self, chunk_key: str) -> None:
        """Forget ``chunk_key``; unknown keys are ignored."""

    def discard(self, chunk_key: str) -> None:
        """Synchronous removal used by eviction; defaults to a scheduled remove."""
        import asyncio

        try:
            loop = asyncio.get_running_loop()
        except RuntimeError:
            asyncio.run(self.remove(chunk_key))
        else:
            loop.create_task(self.remove(chunk_key))
