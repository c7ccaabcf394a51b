"""Byte layout of slots, layers and chunks in the store, and the TP head map.

Container (identical to the reference, ``daser/connector/daser_connector.py:488,
548,608,626`` and ``docs/design/components.md:21-55``): the store is a flat file
of ``total_slots`` fixed-size slots; a slot holds one KV block
(``block_tokens`` tokens) for **all** layers, layer-major; a chunk is
``ceil(tokens / block_tokens)`` contiguous slots.  Byte offset of
``(slot i, layer l)`` of a chunk = ``(start_slot + i) * slot_size + l * layer_size``.

Layer region, ``raw`` codec (reference-compatible): the KV dtype bytes of
``[K|V][token][head][dim]``.

Layer region, ``fp8b16`` codec (no counterpart in the reference): e4m3 payload
``[K|V][token][head][dim]`` (1 byte per element) followed by fp32 scales
``[K|V][token][head][dim/16]``; 1.25 bytes per element.

Chunks are stored with **all** KV heads (TP-agnostic) so a chunk written at
one tensor-parallel degree restores at any other; rank ``r`` of ``tp`` owns
heads ``[r*H/tp, (r+1)*H/tp)`` (or a replica of head ``r*H//tp`` when
``tp > H``).
"""

from __future__ import annotations

from dataclasses import dataclass

from daser_b200.config import CODEC_FP8B16, CODEC_RAW, FP8_GROUP, DaserConfig


@dataclass(frozen=True)
class KVGeometry:
    num_layers: int
    num_kv_heads: int
    head_dim: int
    block_tokens: int = 16
    dtype_bytes: int = 2
    codec: str = CODEC_RAW

    @classmethod
    def from_config(cls, cfg: DaserConfig) -> "KVGeometry":
        return cls(
            cfg.num_layers,
            cfg.num_kv_heads,
            cfg.head_dim,
            cfg.block_tokens,
            cfg.dtype_bytes,
            cfg.codec,
        )

    def __post_init__(self) -> None:
        if min(self.num_layers, self.num_kv_heads, self.head_dim, self.block_tokens) <= 0:
            raise ValueError("geometry fields must be positive")
        if self.codec not in (CODEC_RAW, CODEC_FP8B16):
            raise ValueError(f"unknown codec {self.codec!r}")
        if self.codec == CODEC_FP8B16 and self.head_dim % FP8_GROUP:
            raise ValueError("fp8b16 needs head_dim to be a multiple of 16")

    # element counts ---------------------------------------------------------
    @property
    def elems_per_kv(self) -> int:
        """Elements of K (or of V) in one layer of one block."""
        return self.block_tokens * self.num_kv_heads * self.head_dim

    @property
    def elems_per_layer(self) -> int:
        return 2 * self.elems_per_kv

    # byte sizes ----------------------------------------------------------------
    @property
    def payload_bytes_per_layer(self) -> int:
        if self.codec == CODEC_RAW:
            return self.elems_per_layer * self.dtype_bytes
        return self.elems_per_layer

    @property
    def scale_bytes_per_layer(self) -> int:
        if self.codec == CODEC_RAW:
            return 0
        return self.elems_per_layer // FP8_GROUP * 4

    @property
    def layer_size(self) -> int:
        return self.payload_bytes_per_layer + self.scale_bytes_per_layer

    @property
    def slot_size(self) -> int:
        return self.layer_size * self.num_layers

    # offsets ----------------------------------------------------------------------
    def slots_for(self, token_count: int) -> int:
        return -(-token_count // self.block_tokens)

    def slot_offset(self, slot: int) -> int:
        return slot * self.slot_size

    def layer_offset(self, start_slot: int, slot_i: int, layer: int) -> int:
        return (start_slot + slot_i) * self.slot_size + layer * self.layer_size

    def with_codec(self, codec: str) -> "KVGeometry":
        return KVGeometry(
            self.num_layers,
            self.num_kv_heads,
            self.head_dim,
            self.block_tokens,
            self.dtype_bytes,
            codec,
        )


def tp_head_range(num_kv_heads: int, tp: int, rank: int) -> tuple[int, int]:
    """``(first_head, count)`` of the KV heads rank ``rank`` keeps.

    With more ranks than KV heads the heads are replicated: ranks
    ``[h*tp/H, (h+1)*tp/H)`` all keep head ``h``.
    """
    if not 0 <= rank < tp:
        raise ValueError("rank outside [0, tp)")
    if tp <= num_kv_heads:
        if num_kv_heads % tp:
            raise ValueError("num_kv_heads must be divisible by tp")
        per = num_kv_heads // tp
        return rank * per, per
    if tp % num_kv_heads:
        raise ValueError("tp must be a multiple of num_kv_heads")
    return rank // (tp // num_kv_heads), 1


def owner_rank(chunk_key: str, tp: int) -> int:
    """The rank that does the NVMe IO for ``chunk_key`` (spreads PCIe/NVMe load)."""
    return int(chunk_key[-8:], 16) % tp if tp > 1 else 0
