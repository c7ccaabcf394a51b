"""Entry points of the bandwidth-bound model kernels (``ops/csrc/elementwise.cu``)."""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from daser_b200.ops import _lib
from daser_b200.ops.kv_ops import PagedKVPool


class TpSync(C.Structure):
    """Mirror of ``DaserTpSync`` (``ops/csrc/elementwise.cu``)."""

    _fields_ = [
        ("wait_counter", C.c_void_p),
        ("wait_target", C.c_uint32),
        ("done_counter", C.c_void_p),
        ("done_target", C.c_uint32),
        ("signal", C.c_void_p * _lib.MAX_RANKS),
        ("n_signal", C.c_int32),
        ("status", C.c_void_p),
        ("wait_base", C.c_void_p),
        ("done_base", C.c_void_p),
        ("mc_x", C.c_void_p),
    ]


def wait_flags(flags_ptr: int, n: int, target: int, status: Optional[torch.Tensor] = None,
               base_ptr: Optional[int] = None) -> None:
    """Stream-ordered, bounded wait until ``flags[0..n) >= target (+ *base)`` (one-thread kernel)."""
    _lib.check(
        _lib.lib().daser_wait_flags(C.c_void_p(flags_ptr), n, C.c_uint32(target), C.c_void_p(base_ptr),
                                    C.c_void_p(status.data_ptr()) if status is not None else None,
                                    _lib.stream_ptr()),
        "wait_flags",
    )


def signal_flags(flag_ptrs: Sequence[int], value: int, stream=None) -> None:
    """Stream-ordered: after everything queued before it (stores into peers' memory included) is
    visible system-wide, write ``value`` into each of ``flag_ptrs`` (device addresses, possibly in
    peers' memory).  The counterpart of :func:`wait_flags`."""
    arr = (C.c_uint64 * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    _lib.check(_lib.lib().daser_signal_flags(arr, len(flag_ptrs), C.c_uint32(value & 0xFFFFFFFF),
                                             _lib.stream_ptr(stream)), "signal_flags")


def tp_pick_token(best_val: torch.Tensor, best_idx: torch.Tensor, n: int, rank: int, tp: int, cap: int,
                  table_ptrs: Sequence[int], counter_ptrs: Sequence[int], epoch: torch.Tensor,
                  status: Optional[torch.Tensor], out_idx: torch.Tensor) -> None:
    """The tensor-parallel sample in one kernel: push this rank's per-row candidates (``best_val``
    float32, ``best_idx`` int32: the best of its vocabulary shard) into every rank's table, publish
    an arrival in every rank's counter, wait (bounded) for all ``tp`` arrivals here, and write the
    winning index per row into ``out_idx``.  ``table_ptrs[r]`` = rank r's table of
    ``2 * tp * 2 * cap`` floats, ``counter_ptrs[r]`` its arrival counter, ``epoch`` this rank's
    count of consumed arrivals (int32[1], device)."""
    assert best_val.dtype == torch.float32 and best_idx.dtype == torch.int32 and out_idx.dtype == torch.int32
    tables = (C.c_uint64 * tp)(*[int(x) for x in table_ptrs])
    counters = (C.c_uint64 * tp)(*[int(x) for x in counter_ptrs])
    _lib.check(
        _lib.lib().daser_tp_pick_token(C.c_void_p(best_val.data_ptr()), C.c_void_p(best_idx.data_ptr()), n, rank, tp,
                                       cap, tables, counters, C.c_void_p(epoch.data_ptr()),
                                       C.c_void_p(status.data_ptr()) if status is not None else None,
                                       C.c_void_p(out_idx.data_ptr()), _lib.stream_ptr()),
        "tp_pick_token",
    )


def advance_epochs(epochs: torch.Tensor, d0: int, d1: int, d2: int) -> None:
    """``epochs[0:3] += (d0, d1, d2)`` on the stream (see ``parallel/tp.py``)."""
    _lib.check(
        _lib.lib().daser_advance_epochs(C.c_void_p(epochs.data_ptr()), C.c_uint32(d0), C.c_uint32(d1),
                                        C.c_uint32(d2), _lib.stream_ptr()),
        "advance_epochs",
    )


def _is_f32(t: torch.Tensor) -> int:
    assert t.dtype in (torch.float32, torch.bfloat16)
    return int(t.dtype == torch.float32)


def add_rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    eps: float = 1e-5,
    zero_after: bool = False,
    out_ptrs: Optional[Sequence[int]] = None,
    out_row_offset: int = 0,
    tp_sync: Optional[TpSync] = None,
    n_partials: int = 1,
    partial_stride: int = 0,
) -> Optional[torch.Tensor]:
    """``out = rmsnorm(x + residual) * weight``; ``residual`` is updated in place.

    ``x`` is bf16, or an fp32 accumulator that is zeroed after the read when
    ``zero_after``.  ``out_ptrs`` (raw addresses, possibly peers') replaces ``out`` for the
    all-gather push: each receives the rows at ``out_row_offset``.
    """
    rows, hidden = x.shape
    if out_ptrs is None:
        if out is None:
            out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=x.device)
        out_ptrs = [out.data_ptr()]
    arr = (C.c_void_p * len(out_ptrs))(*out_ptrs)
    _lib.check(
        _lib.lib().daser_add_rmsnorm_tp(
            C.c_void_p(x.data_ptr()), _is_f32(x),
            C.c_void_p(residual.data_ptr()) if residual is not None else None,
            C.c_void_p(weight.data_ptr()), arr, len(out_ptrs), C.c_int64(out_row_offset),
            C.c_int64(rows), hidden, C.c_float(eps), int(zero_after),
            C.byref(tp_sync) if tp_sync is not None else None, n_partials, C.c_int64(partial_stride),
            _lib.stream_ptr(),
        ),
        "add_rmsnorm",
    )
    return out


def rope_kv_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    slot_mapping: torch.Tensor,
    cos_sin: torch.Tensor,
    q_out: torch.Tensor,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    block_tokens: int,
    pool: PagedKVPool,
    layer: int,
    rank: int = 0,
    zero_after: bool = False,
    qk_norm: Optional[tuple[torch.Tensor, torch.Tensor, float]] = None,
) -> None:
    """RoPE on q and k of ``qkv[T, (Hq + 2 Hkv) * D]``; q -> ``q_out``, k/v -> the paged pool.

    ``qk_norm = (q_weight[D], k_weight[D], eps)``: RMSNorm over head_dim on every query and key
    head before the rotation (Qwen3 family)."""
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int64
    pool_c = pool.c_struct()
    if qk_norm is not None:
        qw, kw, eps = qk_norm
        assert qw.dtype == torch.bfloat16 and kw.dtype == torch.bfloat16 and qw.numel() == head_dim == kw.numel()
        _lib.check(
            _lib.lib().daser_rope_kv_write_qknorm(
                C.c_void_p(qkv.data_ptr()), _is_f32(qkv), C.c_int64(qkv.stride(0)),
                C.c_void_p(positions.data_ptr()), C.c_void_p(slot_mapping.data_ptr()),
                C.c_void_p(cos_sin.data_ptr()), int(cos_sin.shape[0]), C.c_void_p(q_out.data_ptr()),
                int(qkv.shape[0]), num_q_heads, num_kv_heads, head_dim, block_tokens,
                C.byref(pool_c), layer, rank, int(zero_after), C.c_void_p(qw.data_ptr()),
                C.c_void_p(kw.data_ptr()), C.c_float(eps), _lib.stream_ptr(),
            ),
            "rope_kv_write_qknorm",
        )
        return
    _lib.check(
        _lib.lib().daser_rope_kv_write(
            C.c_void_p(qkv.data_ptr()), _is_f32(qkv), C.c_int64(qkv.stride(0)),
            C.c_void_p(positions.data_ptr()), C.c_void_p(slot_mapping.data_ptr()),
            C.c_void_p(cos_sin.data_ptr()), int(cos_sin.shape[0]), C.c_void_p(q_out.data_ptr()),
            int(qkv.shape[0]), num_q_heads, num_kv_heads, head_dim, block_tokens,
            C.byref(pool_c), layer, rank, int(zero_after), _lib.stream_ptr(),
        ),
        "rope_kv_write",
    )


def swiglu(x: torch.Tensor, out: Optional[torch.Tensor] = None, zero_after: bool = False,
           block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` for ``x[T, 2I]`` (bf16 or fp32 accumulators): ``x = [gate | up]``, or with
    ``block`` > 0 blocks of ``block`` gate columns followed by the matching up columns."""
    T, two_i = x.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=torch.bfloat16, device=x.device)
    _lib.check(
        _lib.lib().daser_swiglu(C.c_void_p(x.data_ptr()), _is_f32(x), C.c_void_p(out.data_ptr()),
                                C.c_int64(T), inter, int(zero_after), int(block), _lib.stream_ptr()),
        "swiglu",
    )
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None,
              vocab_begin: int = 0) -> torch.Tensor:
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16
    T, hidden = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, hidden), dtype=torch.bfloat16, device=table.device)
    _lib.check(
        _lib.lib().daser_embedding(C.c_void_p(ids.data_ptr()), C.c_void_p(table.data_ptr()),
                                   C.c_void_p(out.data_ptr()), C.c_int64(T), hidden, vocab_begin,
                                   int(table.shape[0]), _lib.stream_ptr()),
        "embedding",
    )
    return out


def argmax(logits: torch.Tensor, best_val: torch.Tensor, best_idx: torch.Tensor,
           index_offset: int = 0, zero_after: bool = False,
           sampling: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> None:
    """Per row: the index (plus ``index_offset``) and value of the largest logit.

    ``sampling = (inv_temp float32[rows], seeds int64[rows])`` draws from ``softmax(logits * inv_temp)``
    instead, by the Gumbel-max rule (``best_val`` is then the perturbed maximum, which is what
    tensor-parallel ranks compare); rows with ``inv_temp == 0`` stay greedy."""
    rows, n = logits.shape
    if sampling is not None:
        inv_temp, seeds = sampling
        assert inv_temp.dtype == torch.float32 and seeds.dtype == torch.int64
        assert inv_temp.numel() >= rows and seeds.numel() >= rows
        _lib.check(
            _lib.lib().daser_argmax_sample(C.c_void_p(logits.data_ptr()), _is_f32(logits), C.c_int64(logits.stride(0)),
                                           rows, n, index_offset, C.c_void_p(best_val.data_ptr()),
                                           C.c_void_p(best_idx.data_ptr()), int(zero_after),
                                           C.c_void_p(inv_temp.data_ptr()), C.c_void_p(seeds.data_ptr()),
                                           _lib.stream_ptr()),
            "argmax_sample",
        )
        return
    _lib.check(
        _lib.lib().daser_argmax(C.c_void_p(logits.data_ptr()), _is_f32(logits), C.c_int64(logits.stride(0)),
                                rows, n, index_offset, C.c_void_p(best_val.data_ptr()),
                                C.c_void_p(best_idx.data_ptr()), int(zero_after), _lib.stream_ptr()),
        "argmax",
    )
