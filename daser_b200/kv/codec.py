"""CPU reference for the block-scaled fp8 codec, RoPE and slot packing.

This is the oracle for the CUDA kernels (``ops/csrc/kv_codec.cu``,
``kv_restore.cu``, ``kv_save.cu``) and the implementation used by the CPU-only
engine.  The reference stores KV raw and has no codec, RoPE or repacking code
(``daser/connector/daser_connector.py:625-632`` is a byte copy), so everything
here is new.

fp8b16: groups of 16 consecutive ``dim`` elements share one fp32 scale
``s = absmax / 448`` (``s = 1`` for an all-zero group); the payload is
``rne_e4m3(x * (448 / absmax))``.  Dequantisation is ``q * s``.  All arithmetic
is IEEE fp32 so the CUDA kernels reproduce it bit for bit.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from daser_b200.config import CODEC_RAW, FP8_GROUP
from daser_b200.kv.layout import KVGeometry

E4M3_MAX = 448.0


def quantize_fp8b16(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``x[..., D]`` (any float dtype) -> (uint8 e4m3 payload ``[..., D]``, fp32 scales ``[..., D/16]``)."""
    if x.shape[-1] % FP8_GROUP:
        raise ValueError("last dimension must be a multiple of 16")
    xf = x.detach().to(torch.float32)
    g = xf.reshape(*xf.shape[:-1], xf.shape[-1] // FP8_GROUP, FP8_GROUP)
    absmax = g.abs().amax(dim=-1, keepdim=True)
    nz = absmax > 0
    safe = torch.where(nz, absmax, torch.ones_like(absmax))
    # tensor / tensor so both are true IEEE divisions (scalar operands make torch multiply
    # by a reciprocal, which rounds differently from the kernels' div.rn)
    top = torch.full_like(safe, E4M3_MAX)
    inv = torch.where(nz, torch.div(top, safe), torch.ones_like(absmax))
    scale = torch.where(nz, torch.div(safe, top), torch.ones_like(absmax))
    q = (g * inv).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(x.shape), scale.squeeze(-1).contiguous()


def dequantize_fp8b16(
    payload: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.float32
) -> torch.Tensor:
    q = payload.view(torch.float8_e4m3fn).to(torch.float32)
    g = q.reshape(*q.shape[:-1], q.shape[-1] // FP8_GROUP, FP8_GROUP)
    return (g * scales.to(torch.float32).unsqueeze(-1)).reshape(payload.shape).to(dtype)


# -- RoPE ---------------------------------------------------------------------------


def rope_cos_sin(
    positions: torch.Tensor, inv_freq: Sequence[float] | torch.Tensor
) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of ``positions[:, None] * inv_freq[None, :]`` computed in fp64, returned fp32."""
    inv = torch.as_tensor(inv_freq, dtype=torch.float64)
    ang = positions.to(torch.float64).reshape(-1, 1) * inv.reshape(1, -1)
    return ang.cos().to(torch.float32), ang.sin().to(torch.float32)


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half (NeoX) RoPE.  ``x[T, H, D]``, ``cos/sin[T, D/2]`` (or ``[1, D/2]``)."""
    half = x.shape[-1] // 2
    xf = x.to(torch.float32)
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def rope_delta_rotate(
    k: torch.Tensor, delta: int, inv_freq: Sequence[float] | torch.Tensor
) -> torch.Tensor:
    """Move already-rotated keys ``k[..., H, D]`` by ``delta`` positions."""
    if delta == 0:
        return k.to(torch.float32)
    cos, sin = rope_cos_sin(torch.tensor([delta]), inv_freq)
    flat = k.reshape(-1, k.shape[-2], k.shape[-1])
    return rope_rotate(flat, cos, sin).reshape(k.shape)


# -- slot images ------------------------------------------------------------------------


def pack_layer(geo: KVGeometry, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``k, v`` of shape ``[block_tokens, H, D]`` -> the layer's bytes (uint8, 1-D)."""
    kv = torch.stack([k, v])  # [2, B, H, D]
    if geo.codec == CODEC_RAW:
        want = {2: (torch.bfloat16, torch.float16), 4: (torch.float32,), 1: (torch.uint8,)}
        if kv.dtype not in want[geo.dtype_bytes]:
            raise ValueError(f"dtype {kv.dtype} does not match dtype_bytes={geo.dtype_bytes}")
        return kv.contiguous().view(torch.uint8).reshape(-1)
    payload, scales = quantize_fp8b16(kv)
    return torch.cat([payload.reshape(-1), scales.reshape(-1).view(torch.uint8)])


def unpack_layer(
    geo: KVGeometry, raw: torch.Tensor, dtype: torch.dtype = torch.float32
) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_layer`; returns ``k, v`` ``[block_tokens, H, D]`` in ``dtype``."""
    shape = (2, geo.block_tokens, geo.num_kv_heads, geo.head_dim)
    raw = raw.reshape(-1)
    if raw.numel() != geo.layer_size:
        raise ValueError(f"layer region has {raw.numel()} bytes, expected {geo.layer_size}")
    if geo.codec == CODEC_RAW:
        src = {2: torch.bfloat16, 4: torch.float32}[geo.dtype_bytes]
        if dtype in (torch.float16,) and geo.dtype_bytes == 2:
            src = torch.float16
        kv = raw.contiguous().view(src).reshape(shape).to(dtype)
    else:
        n = geo.payload_bytes_per_layer
        payload = raw[:n].reshape(shape)
        scales = raw[n:].contiguous().view(torch.float32).reshape(*shape[:-1], -1)
        kv = dequantize_fp8b16(payload, scales, dtype)
    return kv[0], kv[1]


def pack_slot(geo: KVGeometry, ks: Sequence[torch.Tensor], vs: Sequence[torch.Tensor]) -> torch.Tensor:
    """One slot image from per-layer ``k, v`` blocks."""
    return torch.cat([pack_layer(geo, k, v) for k, v in zip(ks, vs)])


def restore_slot_reference(
    geo: KVGeometry,
    slot: torch.Tensor,
    delta: int,
    inv_freq: Sequence[float] | torch.Tensor,
    head_range: Optional[tuple[int, int]] = None,
    dtype: torch.dtype = torch.float32,
) -> list[tuple[torch.Tensor, torch.Tensor]]:
    """Oracle for the restore kernel on one slot: per layer ``(k_rotated, v)``.

    ``head_range=(first, count)`` selects one TP rank's heads.
    """
    out = []
    for layer in range(geo.num_layers):
        raw = slot[layer * geo.layer_size : (layer + 1) * geo.layer_size]
        k, v = unpack_layer(geo, raw, torch.float32)
        k = rope_delta_rotate(k, delta, inv_freq)
        if head_range is not None:
            h0, hn = head_range
            k, v = k[:, h0 : h0 + hn], v[:, h0 : h0 + hn]
        out.append((k.to(dtype), v.to(dtype)))
    return out
