"""tcgen05 GEMM entry points (``ops/csrc/gemm.cu``).

``linear(x, w)`` computes ``x @ w.T`` for bf16 ``x[M, K]`` and a Linear weight
``w[N, K]``.  Two output forms:

* ``out`` bf16 ``[M, N]`` (no split-K), or
* ``acc`` fp32 ``[M, N]`` accumulated with ``red.global.add`` (split-K and/or
  reduce-scatter: ``owners`` lists per-rank accumulation buffers, each holding
  ``rows_per_owner`` rows).

``plan_tiles`` picks the N tile and the K split so that at least one CTA per SM streams
weights when M is small.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from daser_b200.ops import _lib
from daser_b200.ops._lib import Gemm

NUM_SMS = 148
EPI_STORE_BF16 = 0
EPI_REDUCE_F32 = 1
EPI_SPLITK_SCATTER = 2
EPI_SWIGLU_BF16 = 3
EPI_QKV_ROPE = 4
GATE_UP_BLOCK = 64  # gate/up rows are interleaved in blocks of this many (half of a 128-row tile)


def plan_tiles(M: int, N: int, K: int, allow_split: bool = True) -> tuple[int, int]:
    """(block_n, k_splits) for a GEMM of this shape."""
    m_tiles = -(-M // 128)
    if m_tiles * -(-N // 256) >= 2 * NUM_SMS:
        return 256, 1  # compute-bound: the biggest tile, no split
    block_n = 128
    tiles = m_tiles * -(-N // block_n)
    if not allow_split or tiles >= NUM_SMS:
        return block_n, 1
    kb = -(-K // 64)
    # aim for ~2 CTAs per SM, each with at least 4 K blocks
    want = max(1, (2 * NUM_SMS) // tiles)
    return block_n, max(1, min(want, kb // 4 if kb >= 4 else 1))


def expected_arrivals(M: int, N: int, block_n: int, k_splits: int, rows_per_owner: int, n_owners: int,
                      K: int) -> list[int]:
    """Arrival-counter increments each owner receives from ONE rank's GEMM launch.

    Mirrors the kernel: every CTA (one 128-row tile) bumps each owner its rows touch, once
    per (n tile, non-empty k split).  The split-K scatter epilogue signals only from the CTA
    that completes a tile: pass ``k_splits=1`` for it.
    """
    kb_total = -(-K // 64)
    kb_per = -(-kb_total // k_splits)
    live_splits = sum(1 for z in range(k_splits) if z * kb_per < kb_total)
    n_tiles = -(-N // block_n)
    counts = [0] * n_owners
    for m0 in range(0, M, 128):
        o0 = m0 // rows_per_owner
        o1 = min(m0 + 127, M - 1) // rows_per_owner
        for o in range(o0, o1 + 1):
            counts[o] += n_tiles * live_splits
    return counts


def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    acc: Optional[torch.Tensor] = None,
    owners: Optional[Sequence[int]] = None,
    rows_per_owner: Optional[int] = None,
    arrive: Optional[Sequence[int]] = None,
    block_n: Optional[int] = None,
    k_splits: Optional[int] = None,
    status: Optional[torch.Tensor] = None,
    gate_flags: Optional[int] = None,
    gate_target: int = 0,
    gate_rows: int = 0,
    gate_base: Optional[int] = None,
    scatter_bf16: bool = False,
    dst_row_offset: int = 0,
    work: Optional[torch.Tensor] = None,
    tile_counters: Optional[torch.Tensor] = None,
    ldc: Optional[int] = None,
    broadcast: bool = False,
    signal_all: bool = False,
    stream=None,
) -> torch.Tensor:
    assert x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
    assert x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    if scatter_bf16:
        # reduce-scatter, bf16 form: plain stores into slot `dst_row_offset / rows_per_owner` of
        # every owner's receive buffer; no split-K (stores cannot accumulate)
        assert owners is not None and rows_per_owner is not None and ldc is not None
        g = Gemm()
        g.a, g.b = x.data_ptr(), w.data_ptr()
        g.lda, g.ldb, g.ldc = x.stride(0), w.stride(0), ldc
        g.M, g.N, g.K = x.shape[0], w.shape[0], x.shape[1]
        g.block_n, g.k_splits, g.epilogue = block_n or 64, 1, EPI_STORE_BF16
        if work is not None and (k_splits or 1) > 1:
            # split-K into the local fp32 work buffer; the last CTA of a tile scatters the sum
            assert tile_counters is not None and work.dtype == torch.float32
            g.k_splits, g.epilogue = k_splits, EPI_SPLITK_SCATTER
            g.work, g.work_ld, g.tile_counters = work.data_ptr(), work.stride(0), tile_counters.data_ptr()
        g.n_owners, g.rows_per_owner, g.dst_row_offset = len(owners), rows_per_owner, dst_row_offset
        # broadcast: the one-shot all-reduce form.  Every rank receives this rank's whole partial
        # (rows are not partitioned: row r lands at dst_row_offset + r of every owner's buffer)
        g.bcast = 1 if broadcast else 0
        # signal_all: the partial stays in this rank's own buffer (owners[0]); every rank's arrival
        # counter is bumped, after which peers read the sum through the NVLink multicast mapping
        if signal_all:
            assert not broadcast
            g.bcast = 2
        for i, ptr in enumerate(owners):
            g.c[i] = ptr
        for i, ptr in enumerate(arrive or []):
            g.arrive[i] = ptr
        g.status = status.data_ptr() if status is not None else None
        _lib.check(_lib.lib().daser_gemm(C.byref(g), _lib.stream_ptr(stream)), "gemm")
        return None  # type: ignore[return-value]
    reduce = acc is not None or owners is not None
    bn, ks = plan_tiles(M, N, K, allow_split=reduce)
    bn = block_n or bn
    ks = k_splits or ks
    g = Gemm()
    g.a, g.b = x.data_ptr(), w.data_ptr()
    g.lda, g.ldb = x.stride(0), w.stride(0)
    g.M, g.N, g.K = M, N, K
    g.block_n, g.k_splits = bn, ks
    g.status = status.data_ptr() if status is not None else None
    g.gate_flags, g.gate_target, g.gate_rows, g.gate_base = gate_flags, gate_target, gate_rows, gate_base
    if reduce:
        g.epilogue = EPI_REDUCE_F32
        if owners is None:
            assert acc is not None and acc.dtype == torch.float32 and acc.stride(1) == 1
            owners, rows_per_owner = [acc.data_ptr()], max(M, 1)
            g.ldc = acc.stride(0)
        else:
            assert rows_per_owner is not None and ldc is not None
            g.ldc = ldc
        g.n_owners, g.rows_per_owner = len(owners), rows_per_owner
        for i, ptr in enumerate(owners):
            g.c[i] = ptr
        if arrive is not None:
            for i, ptr in enumerate(arrive):
                g.arrive[i] = ptr
        result = acc
    else:
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1
        g.epilogue = EPI_STORE_BF16
        g.ldc = out.stride(0)
        g.n_owners, g.rows_per_owner = 1, max(M, 1)
        g.c[0] = out.data_ptr()
        result = out
    _lib.check(_lib.lib().daser_gemm(C.byref(g), _lib.stream_ptr(stream)), "gemm")
    return result


def can_fuse_qkv_rope(head_dim: int, qk_norm: bool) -> bool:
    """The QKV projection can end in RoPE + the paged KV write when a 128-column tile is one head
    and no per-head norm sits between the projection and the rotation."""
    return head_dim == 128 and not qk_norm


def linear_qkv_rope(x: torch.Tensor, wqkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                    cos_sin: torch.Tensor, q_out: torch.Tensor, hq: int, hkv: int, block_tokens: int, pool, layer: int,
                    rank: int, work: torch.Tensor, tile_counters: torch.Tensor, k_splits: Optional[int] = None,
                    status: Optional[torch.Tensor] = None, gate_flags: Optional[int] = None, gate_target: int = 0,
                    gate_rows: int = 0, gate_base: Optional[int] = None, stream=None) -> None:
    """``x @ wqkv.T`` with RoPE and the KV-cache write as the GEMM's epilogue.

    Query heads land rotated in ``q_out`` (bf16 ``[T, hq, 128]``); key heads are rotated and, like
    the value heads, quantised into ``pool`` at ``slot_mapping``.  ``work`` (fp32 ``[>= T, N]``,
    zero) and ``tile_counters`` (int32, zero) serve the split-K case and come back zeroed."""
    assert x.dtype == torch.bfloat16 and wqkv.dtype == torch.bfloat16 and x.stride(1) == 1 and wqkv.stride(1) == 1
    M, K = x.shape
    N = wqkv.shape[0]
    assert N == (hq + 2 * hkv) * 128 and q_out.dtype == torch.bfloat16 and q_out.is_contiguous()
    assert work.dtype == torch.float32 and work.shape[1] >= N and work.shape[0] >= M
    _, ks = plan_tiles(M, N, K, allow_split=True)
    ks = k_splits or ks
    g = Gemm()
    g.a, g.b = x.data_ptr(), wqkv.data_ptr()
    g.lda, g.ldb, g.ldc = x.stride(0), wqkv.stride(0), N
    g.M, g.N, g.K = M, N, K
    g.block_n, g.k_splits, g.epilogue = 128, ks, EPI_QKV_ROPE
    g.n_owners, g.rows_per_owner = 1, max(M, 1)
    g.work, g.work_ld, g.tile_counters = work.data_ptr(), work.stride(0), tile_counters.data_ptr()
    g.status = status.data_ptr() if status is not None else None
    g.gate_flags, g.gate_target, g.gate_rows, g.gate_base = gate_flags, gate_target, gate_rows, gate_base
    pool_c = pool.c_struct()
    g.rope_positions, g.rope_slot_mapping = positions.data_ptr(), slot_mapping.data_ptr()
    g.rope_cos_sin, g.rope_q_out = cos_sin.data_ptr(), q_out.data_ptr()
    g.rope_pool = C.addressof(pool_c)
    g.rope_max_pos, g.rope_hq, g.rope_hkv = int(cos_sin.shape[0]), hq, hkv
    g.rope_block_tokens, g.rope_layer, g.rope_rank = block_tokens, layer, rank
    _lib.check(_lib.lib().daser_gemm(C.byref(g), _lib.stream_ptr(stream)), "gemm_qkv_rope")


def interleave_gate_up(w_gate_up: torch.Tensor, block: int = GATE_UP_BLOCK) -> torch.Tensor:
    """``[gate rows | up rows]`` -> blocks of ``block`` gate rows followed by the matching up rows.

    With this row order every ``2 * block``-row GEMM tile holds the gate and the up values of
    the same outputs, which is what lets the activation run in the GEMM epilogue.
    """
    two_i, hidden = w_gate_up.shape
    inter = two_i // 2
    assert inter % block == 0
    return (w_gate_up.view(2, inter // block, block, hidden).transpose(0, 1).reshape(two_i, hidden).contiguous())


def can_fuse_swiglu(M: int, two_i: int, K: int, split_ok: bool = False) -> bool:
    """True when the gate/up GEMM of this shape can apply the activation itself: 128-row tiles, and
    either unsplit (one CTA per tile sees the whole K range) or, with ``split_ok``, split-K with the
    tile's last CTA finishing from the fp32 work buffer."""
    bn, ks = plan_tiles(M, two_i, K, allow_split=True)
    return (ks == 1 or split_ok) and bn == 128 and two_i % 128 == 0


def linear_swiglu(x: torch.Tensor, w_gate_up_il: torch.Tensor, out: torch.Tensor,
                  status: Optional[torch.Tensor] = None, gate_flags: Optional[int] = None, gate_target: int = 0,
                  gate_rows: int = 0, gate_base: Optional[int] = None, stream=None, k_splits: int = 1,
                  work: Optional[torch.Tensor] = None, tile_counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` in one kernel; ``w_gate_up_il`` is :func:`interleave_gate_up` order.
    ``k_splits > 1`` needs ``work`` (fp32 ``[>= M, N]``, zero) and ``tile_counters`` (zero); both come back zeroed."""
    assert x.dtype == torch.bfloat16 and w_gate_up_il.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    M, K = x.shape
    N = w_gate_up_il.shape[0]
    assert out.shape[0] >= M and out.shape[1] == N // 2 and out.stride(1) == 1
    g = Gemm()
    g.a, g.b = x.data_ptr(), w_gate_up_il.data_ptr()
    g.lda, g.ldb, g.ldc = x.stride(0), w_gate_up_il.stride(0), out.stride(0)
    g.M, g.N, g.K = M, N, K
    g.block_n, g.k_splits, g.epilogue = 2 * GATE_UP_BLOCK, max(1, k_splits), EPI_SWIGLU_BF16
    if k_splits > 1:
        assert work is not None and tile_counters is not None and work.dtype == torch.float32
        assert work.shape[0] >= M and work.shape[1] >= N
        g.work, g.work_ld, g.tile_counters = work.data_ptr(), work.stride(0), tile_counters.data_ptr()
    g.n_owners, g.rows_per_owner = 1, max(M, 1)
    g.c[0] = out.data_ptr()
    g.status = status.data_ptr() if status is not None else None
    g.gate_flags, g.gate_target, g.gate_rows, g.gate_base = gate_flags, gate_target, gate_rows, gate_base
    _lib.check(_lib.lib().daser_gemm(C.byref(g), _lib.stream_ptr(stream)), "gemm_swiglu")
    return out
