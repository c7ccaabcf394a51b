"""Constant position offset.

Capability parity: ``daser/position/fixed_offset.py:11-50``.
"""

from __future__ import annotations

from daser_b200.position.base import PositionEncoder
from daser_b200.server.metadata_store import ChunkMeta


class FixedOffsetEncoder(PositionEncoder):
    def __init__(self, fixed_offset: int = 0) -> None:
        self._offset = int(fixed_offset)

    def assign_offset(self, chunk_key: str, token_count: int) -> int:
        return self._offset

    def get_offset(self, meta: ChunkMeta) -> int:
        return meta.pos_offset
