"""One configuration schema for server, service and connector.

Capability parity: ``daser/config.py:7-75`` (``DaserConfig`` and
``resolved_slot_size``).  The reference keeps three uncoordinated surfaces
(dataclass, two CLIs, connector extra-config) that must be kept equal by hand;
here every surface is built from this dataclass and the connector verifies
the geometry against the server with the ``hello`` RPC
(:meth:`DaserConfig.geometry`).

New fields (no counterpart in the reference): ``codec`` selects the slot
payload encoding (``raw`` = byte-identical to the reference container,
``fp8b16`` = e4m3 payload + one fp32 scale per 16 elements), ``tp_size``
records the tensor-parallel degree the chunks were written at (chunks are
stored TP-agnostic so this is informational), and the RoPE parameters used by
the position re-encoder.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any

CODEC_RAW = "raw"
CODEC_FP8B16 = "fp8b16"
CODECS = (CODEC_RAW, CODEC_FP8B16)
FP8_GROUP = 16  # elements that share one fp32 scale in the fp8b16 codec


def codec_bytes_per_elem_num_den(codec: str, dtype_bytes: int) -> tuple[int, int]:
    """Bytes per KV element of ``codec`` as an exact fraction (num, den)."""
    if codec == CODEC_RAW:
        return dtype_bytes, 1
    if codec == CODEC_FP8B16:
        # 1 payload byte + 4 scale bytes per 16 elements = 20/16
        return FP8_GROUP + 4, FP8_GROUP
    raise ValueError(f"unknown codec {codec!r}; expected one of {CODECS}")


@dataclass
class DaserConfig:
    """Top-level configuration.

    ``slot_size == 0`` means "derive from the model geometry":
    ``kv_heads * head_dim * 2 (K and V) * layers * block_tokens * bytes/elem``.
    """

    store_path: str = "/mnt/xfs/daser.store"
    index_path: str = "/mnt/xfs/daser.index"
    total_slots: int = 1024
    slot_size: int = 0
    ipc_socket_path: str = "/tmp/daser.sock"
    log_level: str = "INFO"
    perf_log_enabled: bool = False
    # model geometry (only needed when slot_size == 0)
    num_kv_heads: int = 0
    head_dim: int = 0
    num_layers: int = 0
    block_tokens: int = 16
    dtype_bytes: int = 2
    model_id: str = "default"
    # --- additions -------------------------------------------------------
    codec: str = CODEC_RAW
    tp_size: int = 1
    rope_theta: float = 10000.0
    rope_scaling: dict[str, Any] = field(default_factory=dict)
    snapshot_interval_s: float = 0.0  # 0 = snapshot on clean shutdown only
    io_backend: str = "auto"  # auto | gds | io_uring | posix

    def resolved_slot_size(self) -> int:
        """Slot size in bytes; derived from the geometry when ``slot_size`` is 0.

        Raises ``ValueError`` naming the first missing model parameter.
        """
        if self.slot_size > 0:
            return self.slot_size
        for name in ("num_kv_heads", "head_dim", "num_layers"):
            if getattr(self, name) == 0:
                raise ValueError(
                    f"slot_size is 0 but {name} is also 0; "
                    "provide either slot_size or all model params"
                )
        elems = (
            self.num_kv_heads * self.head_dim * 2 * self.num_layers * self.block_tokens
        )
        num, den = codec_bytes_per_elem_num_den(self.codec, self.dtype_bytes)
        if (elems * num) % den:
            raise ValueError("geometry is not a whole number of fp8 scale groups")
        return elems * num // den

    def layer_size(self) -> int:
        """Bytes of one layer's region inside a slot."""
        if self.num_layers <= 0:
            raise ValueError("num_layers must be set to compute layer_size")
        return self.resolved_slot_size() // self.num_layers

    def geometry(self) -> dict[str, Any]:
        """The fields both ends of the socket must agree on."""
        return {
            "slot_size": self.resolved_slot_size(),
            "block_tokens": self.block_tokens,
            "num_layers": self.num_layers,
            "num_kv_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "dtype_bytes": self.dtype_bytes,
            "codec": self.codec,
            "model_id": self.model_id,
        }

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def geometry_mismatch(mine: dict[str, Any], theirs: dict[str, Any]) -> list[str]:
    """Names of geometry fields that both sides set (non-zero) and disagree on."""
    bad = []
    for key, val in mine.items():
        other = theirs.get(key)
        if other in (None, 0, "") or val in (None, 0, ""):
            continue
        if other != val:
            bad.append(f"{key}: {val!r} != {other!r}")
    return bad
