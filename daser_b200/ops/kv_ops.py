"""Python entry points of the KV kernels: codec, fused restore, fused save.

``PagedKVPool`` describes a paged pool (one per tensor-parallel rank) with explicit
strides, so the kernels never assume an attention backend's layout; the reference
hard-codes FlashAttention's ``(2, num_blocks, block, heads, dim)`` and breaks on the
FlashInfer layout that Blackwell defaults to
(``daser/connector/daser_connector.py:404-408,544-547,627-630``).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from daser_b200.ops import _lib
from daser_b200.ops._lib import KVJob, KVPool


def quantize_fp8b16(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 CUDA tensor ``[..., D]`` -> (uint8 payload same shape, fp32 scales ``[..., D/16]``)."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    payload = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty((*x.shape[:-1], x.shape[-1] // 16), dtype=torch.float32, device=x.device)
    _lib.check(
        _lib.lib().daser_quant_fp8b16(
            C.c_void_p(x.data_ptr()), C.c_void_p(payload.data_ptr()), C.c_void_p(scales.data_ptr()),
            C.c_int64(x.numel()), _lib.stream_ptr(),
        ),
        "quant_fp8b16",
    )
    return payload, scales


def dequantize_fp8b16(payload: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    assert payload.is_cuda and payload.dtype == torch.uint8 and payload.is_contiguous()
    assert scales.dtype == torch.float32 and scales.is_contiguous()
    out = torch.empty(payload.shape, dtype=torch.bfloat16, device=payload.device)
    _lib.check(
        _lib.lib().daser_dequant_fp8b16(
            C.c_void_p(payload.data_ptr()), C.c_void_p(scales.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_int64(payload.numel()), _lib.stream_ptr(),
        ),
        "dequant_fp8b16",
    )
    return out


@dataclass
class PagedKVPool:
    """A paged KV pool as the kernels see it.

    ``payload_ptrs[r]`` / ``scale_ptrs[r]`` are rank ``r``'s base addresses as mapped into
    *this* process (peers' pools are peer-mapped).  Strides are in elements of the payload
    dtype; the scale tensor has the same shape with ``dim / 16`` as its last dimension.
    """

    payload_ptrs: Sequence[int]
    scale_ptrs: Sequence[int]
    stride_layer: int
    stride_block: int
    stride_kv: int
    stride_tok: int
    stride_head: int
    num_blocks: int
    heads_per_rank: int
    is_fp8: bool
    keepalive: list = field(default_factory=list)

    @property
    def n_ranks(self) -> int:
        return len(self.payload_ptrs)

    def c_struct(self) -> KVPool:
        p = KVPool()
        for r, ptr in enumerate(self.payload_ptrs):
            p.payload[r] = ptr
        for r, ptr in enumerate(self.scale_ptrs):
            p.scales[r] = ptr
        p.stride_layer, p.stride_block = self.stride_layer, self.stride_block
        p.stride_kv, p.stride_tok, p.stride_head = self.stride_kv, self.stride_tok, self.stride_head
        p.num_blocks, p.n_ranks = self.num_blocks, self.n_ranks
        p.heads_per_rank, p.pool_is_fp8 = self.heads_per_rank, int(self.is_fp8)
        return p

    @classmethod
    def from_tensors(
        cls,
        payloads: Sequence[torch.Tensor],
        scales: Optional[Sequence[torch.Tensor]] = None,
        layout: str = "LNKHTD",
    ) -> "PagedKVPool":
        """Build from per-rank tensors.

        ``layout`` names the dimension order of each payload tensor with the letters
        L (layer), N (block), K (k/v), T (token), H (head), D (dim), e.g. ``LNKHTD`` for
        the native engine's head-major pool or ``LKNTHD`` for a stack of vLLM
        FlashAttention layers ``(2, num_blocks, block, heads, dim)``.
        """
        t = payloads[0]
        assert len(layout) == t.dim() and layout[-1] == "D" and t.stride(-1) == 1
        st = {ch: t.stride(i) for i, ch in enumerate(layout)}
        sh = {ch: t.shape[i] for i, ch in enumerate(layout)}
        is_fp8 = t.dtype in (torch.uint8, torch.float8_e4m3fn)
        if is_fp8 and scales is None:
            raise ValueError("an fp8 pool needs its scale tensors")
        return cls(
            payload_ptrs=[p.data_ptr() for p in payloads],
            scale_ptrs=[s.data_ptr() for s in scales] if scales is not None else [0] * len(payloads),
            stride_layer=st.get("L", 0),
            stride_block=st["N"],
            stride_kv=st["K"],
            stride_tok=st["T"],
            stride_head=st["H"],
            num_blocks=sh["N"],
            heads_per_rank=sh["H"],
            is_fp8=is_fp8,
            keepalive=[list(payloads), list(scales) if scales is not None else None],
        )


@dataclass
class KVWorkList:
    """Device-side work list of one restore/save launch."""

    slot_ptrs: torch.Tensor  # int64 [n] addresses of slot images
    block_ids: torch.Tensor  # int32 [n]
    deltas: Optional[torch.Tensor] = None  # int32 [n]

    @property
    def n_slots(self) -> int:
        return int(self.block_ids.numel())


def _job(work, geo, image_is_fp8, cos_sin, status, rank=0) -> KVJob:
    j = KVJob()
    j.slot_ptr = work.slot_ptrs.data_ptr()
    j.block_id = work.block_ids.data_ptr()
    j.delta = work.deltas.data_ptr() if work.deltas is not None else None
    j.cos_sin = cos_sin.data_ptr() if cos_sin is not None else None
    j.status = status.data_ptr() if status is not None else None
    j.max_pos = int(cos_sin.shape[0]) if cos_sin is not None else 0
    j.n_slots = work.n_slots
    j.num_layers, j.num_kv_heads = geo.num_layers, geo.num_kv_heads
    j.head_dim, j.block_tokens = geo.head_dim, geo.block_tokens
    j.image_is_fp8 = int(image_is_fp8)
    j.rank = rank
    return j


def kv_restore(work: KVWorkList, geo, pool: PagedKVPool, cos_sin: Optional[torch.Tensor],
               status: Optional[torch.Tensor] = None, stream=None, layer_begin: int = 0,
               layer_count: int = 0) -> None:
    """Slot images -> paged pools of every rank: dequantise, rotate keys by ``deltas``, scatter.

    ``layer_begin`` / ``layer_count`` restrict the launch to a range of layers (0 = through the
    last one): a restore can then run group by group while the storage reads of later layers
    are still in flight and the model already computes on the earlier ones."""
    job = _job(work, geo, geo.codec == "fp8b16", cos_sin, status)
    job.layer_begin, job.layer_count = int(layer_begin), int(layer_count)
    pool_c = pool.c_struct()
    _lib.check(_lib.lib().daser_kv_restore(C.byref(job), C.byref(pool_c), _lib.stream_ptr(stream)), "kv_restore")


def kv_save(work: KVWorkList, geo, pool: PagedKVPool, rank: int = 0,
            status: Optional[torch.Tensor] = None, stream=None) -> None:
    """Rank ``rank``'s blocks -> its head slice of each slot image (compressing for fp8b16)."""
    job = _job(work, geo, geo.codec == "fp8b16", None, status, rank)
    pool_c = pool.c_struct()
    _lib.check(_lib.lib().daser_kv_save(C.byref(job), C.byref(pool_c), _lib.stream_ptr(stream)), "kv_save")


def copy_rows(dst_ptr: int, src_ptr: int, pitch: int, width: int, rows: int, stream=None) -> None:
    """``rows`` runs of ``width`` bytes, ``pitch`` bytes apart on both sides, copied by the copy
    engine on ``stream`` (either side may be pinned host or device memory)."""
    code = _lib.lib().daser_copy_rows(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), C.c_int64(pitch), C.c_int64(width),
                                      C.c_int64(rows), _lib.stream_ptr(stream))
    if code != 0:
        raise _lib.KernelError(f"copy_rows: CUDA error {code}" if code > 0 else "copy_rows: bad argument")


def rope_table(max_pos: int, inv_freq, device) -> torch.Tensor:
    """``[max_pos, D]`` fp32: cos in ``[:, :D/2]``, sin in ``[:, D/2:]`` (angles in fp64)."""
    inv = torch.as_tensor(inv_freq, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(device)
