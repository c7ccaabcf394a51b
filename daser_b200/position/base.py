"""Position encoder plug-in point.

Capability parity: ``daser/position/base.py:10-48`` — ``assign_offset`` at
allocation time and ``get_offset`` at load time.  In the reference the value
is carried through the RPC replies but nothing consumes it; here the worker
turns ``new_position - get_offset(meta)`` into the rotation applied to cached
keys by the restore kernel.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

from daser_b200.server.metadata_store import ChunkMeta


class PositionEncoder(ABC):
    @abstractmethod
    def assign_offset(self, chunk_key: str, token_count: int) -> int:
        """Position of the chunk's first token when its KV was computed."""

    @abstractmethod
    def get_offset(self, meta: ChunkMeta) -> int:
        """Position the stored keys are currently rotated to."""
