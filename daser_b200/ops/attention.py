"""Paged attention over the block-scaled fp8 pool (``ops/csrc/attention.cu``)."""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from daser_b200.ops import _lib
from daser_b200.ops.kv_ops import PagedKVPool

NUM_SMS = 148
MAX_ROW_SPLITS = 262144  # (query rows x KV splits) the split-KV scratch is sized for (135 MB)


TC_MIN_ROWS = 64  # query rows per KV head from which chunked prefill runs on the tcgen05 kernel
TC_KEY_TILE = 64
_tc_enabled = os.environ.get("DASER_ATTN_TC", "1") != "0"


def set_tensor_core_prefill(enabled: bool) -> None:
    """Route chunked prefill to the tcgen05 kernel (default) or to the mma.sync one."""
    global _tc_enabled
    _tc_enabled = bool(enabled)
    _lib.lib().daser_attention_set_tc(1 if enabled else 0)


def tc_status() -> int:
    """Non-zero if a tcgen05 attention CTA ever gave up on a bounded wait (synchronises)."""
    out = C.c_uint32(0)
    _lib.check(_lib.lib().daser_attention_tc_status(C.byref(out)), "attention_tc_status")
    return int(out.value)


def plan_splits(num_seqs: int, kv_heads: int, max_q_len: int, group: int, max_ctx: int,
                block_tokens: int = 16, rows: int = 0) -> tuple[int, int]:
    """(nsplit, split_tokens): enough work items to fill the GPU."""
    if _tc_enabled and max_q_len * group >= TC_MIN_ROWS and 128 % group == 0:
        # tcgen05 kernel: the unit is a CTA of 128 query rows, two per SM, 64 keys per tile
        base_items = num_seqs * kv_heads * -(-max_q_len * group // 128)
        want = max(1, (NUM_SMS * 2) // max(base_items, 1))
        max_splits = max(1, -(-max_ctx // (2 * TC_KEY_TILE)))  # splits of two key tiles at the shortest
        nsplit = max(1, min(want, max_splits, 64))
        if rows > 0:
            nsplit = max(1, min(nsplit, MAX_ROW_SPLITS // rows))
        per = -(-max_ctx // nsplit)
        split_tokens = -(-per // TC_KEY_TILE) * TC_KEY_TILE
        return -(-max_ctx // split_tokens), split_tokens
    row_tiles = -(-max_q_len * group // 16)
    base_items = num_seqs * kv_heads * row_tiles
    # Measured on the batch-64, 4k-32k decode case: 1024-token splits reach 0.80 of the copy
    # bandwidth, 2048 -> 0.78, 8192 -> 0.53, 256 -> 0.69.  So: splits of about 1024 tokens
    # whenever that still yields several waves of warps, never shorter than 256.
    target_items = NUM_SMS * 8 * 4
    if row_tiles > 1:
        # prefill kernel: the work unit is a CTA of four row tiles, three CTAs fit an SM
        base_items = num_seqs * kv_heads * -(-row_tiles // 4)
        target_items = NUM_SMS * 3 * 2
    want = max(1, -(-target_items // max(base_items, 1)))
    by_len = max(1, max_ctx // 1024)
    max_splits = max(1, max_ctx // 256)
    nsplit = max(1, min(max(want, by_len), max_splits, 128))
    if rows > 0:
        nsplit = max(1, min(nsplit, MAX_ROW_SPLITS // rows))
    per = -(-max_ctx // nsplit)
    split_tokens = -(-per // block_tokens) * block_tokens
    nsplit = -(-max_ctx // split_tokens)
    return nsplit, split_tokens


class AttentionWorkspace:
    """Scratch for split-KV partials, grown on demand and reused."""

    def __init__(self, device) -> None:
        self.device = device
        self.part_o: Optional[torch.Tensor] = None
        self.part_lse: Optional[torch.Tensor] = None

    def ensure(self, rows: int, nsplit: int, head_dim: int) -> None:
        need = rows * nsplit
        if self.part_lse is None or self.part_lse.numel() < need:
            self.part_o = torch.empty(need * head_dim, dtype=torch.float32, device=self.device)
            self.part_lse = torch.empty(need, dtype=torch.float32, device=self.device)


def paged_attention(
    q: torch.Tensor,
    out: torch.Tensor,
    pool: PagedKVPool,
    layer: int,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    ctx_lens: torch.Tensor,
    max_q_len: int,
    max_ctx: int,
    num_kv_heads: int,
    softmax_scale: float,
    workspace: AttentionWorkspace,
    rank: int = 0,
    block_tokens: int = 16,
    nsplit: Optional[int] = None,
    split_tokens: Optional[int] = None,
) -> torch.Tensor:
    """``q, out``: bf16 ``[Tq, Hq, D]``; sequences given by ``q_start`` (prefix sums) and ``ctx_lens``.

    The K/V of the new tokens must already be in the pool; row ``t`` of a sequence attends
    keys ``0 .. ctx_len - q_len + t``.
    """
    Tq, Hq, D = q.shape
    num_seqs = ctx_lens.numel()
    assert block_tables.dtype == torch.int32 and q_start.dtype == torch.int32 and ctx_lens.dtype == torch.int32
    if nsplit is None or split_tokens is None:
        nsplit, split_tokens = plan_splits(num_seqs, num_kv_heads, max_q_len, Hq // num_kv_heads, max_ctx, block_tokens)
    if nsplit > 1:
        workspace.ensure(Tq * Hq, nsplit, D)
    pool_c = pool.c_struct()
    po = workspace.part_o.data_ptr() if nsplit > 1 else None
    pl = workspace.part_lse.data_ptr() if nsplit > 1 else None
    _lib.check(
        _lib.lib().daser_paged_attention_fp8(
            C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()), C.c_void_p(po), C.c_void_p(pl),
            C.byref(pool_c), layer, rank, C.c_void_p(block_tables.data_ptr()), int(block_tables.shape[1]),
            C.c_void_p(q_start.data_ptr()), C.c_void_p(ctx_lens.data_ptr()), num_seqs, Tq, max_q_len,
            Hq, num_kv_heads, D, block_tokens, nsplit, split_tokens, C.c_float(softmax_scale),
            _lib.stream_ptr(),
        ),
        "paged_attention_fp8",
    )
    if nsplit > 1:
        _lib.launch_count += 1  # the merge kernel
    return out
