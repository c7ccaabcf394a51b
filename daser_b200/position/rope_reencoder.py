"""RoPE re-encoding policy: where cached keys were rotated, and by how much to move them.

No counterpart in the reference beyond the unused ``pos_offset`` field.  Rotary
embeddings compose additively: a key computed at position ``p`` and rotated by
a further ``d`` positions equals the key computed at ``p + d``.  A chunk whose
KV was produced with its first token at ``pos_offset`` can therefore be placed
with its first token at ``new_start`` by rotating every key by
``new_start - pos_offset`` positions — one delta for the whole chunk.  Values
are position-free.

The encoder also produces the inverse-frequency table (with optional Llama-3
frequency scaling) shared by the CPU oracle and the restore kernel.
"""

from __future__ import annotations

import math
from typing import Any, Optional

from daser_b200.position.base import PositionEncoder
from daser_b200.server.metadata_store import ChunkMeta


def inv_freq_table(
    head_dim: int, theta: float = 10000.0, scaling: Optional[dict[str, Any]] = None
) -> list[float]:
    """``head_dim/2`` inverse frequencies; ``scaling`` follows Llama-3's rule."""
    half = head_dim // 2
    freqs = [theta ** (-(2.0 * i) / head_dim) for i in range(half)]
    if not scaling:
        return freqs
    factor = float(scaling.get("factor", 8.0))
    low = float(scaling.get("low_freq_factor", 1.0))
    high = float(scaling.get("high_freq_factor", 4.0))
    orig = float(scaling.get("original_max_position_embeddings", 8192))
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


class RopeReencoder(PositionEncoder):
    """Chunks are computed at ``base_offset`` and re-rotated on load."""

    def __init__(
        self,
        head_dim: int = 128,
        theta: float = 10000.0,
        scaling: Optional[dict[str, Any]] = None,
        base_offset: int = 0,
    ) -> None:
        self.head_dim = head_dim
        self.theta = theta
        self.scaling = dict(scaling or {})
        self._base = int(base_offset)

    def assign_offset(self, chunk_key: str, token_count: int) -> int:
        return self._base

    def get_offset(self, meta: ChunkMeta) -> int:
        return meta.pos_offset

    def delta(self, meta_or_offset: ChunkMeta | int, new_start: int) -> int:
        """Positions to rotate stored keys by so the chunk starts at ``new_start``."""
        old = (
            meta_or_offset
            if isinstance(meta_or_offset, int)
            else self.get_offset(meta_or_offset)
        )
        return int(new_start) - int(old)

    def inv_freq(self) -> list[float]:
        return inv_freq_table(self.head_dim, self.theta, self.scaling)
