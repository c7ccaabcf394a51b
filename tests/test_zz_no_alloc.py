"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the library cannot call cudaMalloc: a server that froze its device memory
layout at start-up, a latency-critical loop that must not hit an allocation's implicit
synchronisation, or a foreign runtime that only passes raw pointers through the C ABI.  For
them ``daser_paged_attention_fp8_noalloc`` keeps the split-KV scratch inside the library.
This test calls it on two different cases, each twice in a row (every call after the first
finds an earlier call's leftovers in the shared scratch, its own shape's or another's), and
compares each result with the regular entry point, which works in caller-provided scratch.  It lives in a file of its own that sorts last, so a run that
stops at the first failure has already run everything else.
"""

import ctypes as C

import pytest
import torch

from daser_b200.kv import codec

pytestmark = pytest.mark.gpu


def _case(seed, q_lens, ctx_lens, Hq, Hkv):
    from daser_b200.ops import kv_ops

    torch.manual_seed(seed)
    D, B, L = 128, 16, 1
    n_blocks = sum(-(-c // B) for c in ctx_lens) + 2
    kv = torch.randn(L, n_blocks, 2, Hkv, B, D)
    payload, scales = codec.quantize_fp8b16(kv)
    pool = kv_ops.PagedKVPool.from_tensors([payload.cuda()], [scales.cuda()], "LNKHTD")
    max_blocks = max(-(-c // B) for c in ctx_lens)
    tables = torch.zeros(len(q_lens), max_blocks, dtype=torch.int32)
    used = 0
    for s, c in enumerate(ctx_lens):
        nb = -(-c // B)
        tables[s, :nb] = torch.arange(used, used + nb, dtype=torch.int32)
        used += nb
    q = torch.randn(sum(q_lens), Hq, D).to(torch.bfloat16).cuda()
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    return pool, tables.cuda(), q, q_start, ctx


def _call_noalloc(lib, out, pool, tables, q, q_start, ctx, q_lens, Hq, Hkv, nsplit, split_tokens):
    pool_c = pool.c_struct()
    rc = lib.daser_paged_attention_fp8_noalloc(
        C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()), C.byref(pool_c), 0, 0,
        C.c_void_p(tables.data_ptr()), int(tables.shape[1]), C.c_void_p(q_start.data_ptr()),
        C.c_void_p(ctx.data_ptr()), len(q_lens), int(q.shape[0]), max(q_lens), Hq, Hkv, 128, 16,
        nsplit, split_tokens, C.c_float(128**-0.5), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    from daser_b200.ops import _lib, attention

    lib = _lib.lib()
    cases = [
        (11, [1, 1, 1], [900, 300, 1500], 16, 2, 4, 384),  # decode, 4 KV splits
        (12, [6], [700], 8, 1, 3, 240),                     # short prefill over a context, 3 splits
    ]
    for seed, q_lens, ctx_lens, Hq, Hkv, nsplit, split_tokens in cases:
        pool, tables, q, q_start, ctx = _case(seed, q_lens, ctx_lens, Hq, Hkv)
        ref = torch.zeros_like(q)
        attention.paged_attention(q, ref, pool, 0, tables, q_start, ctx, max(q_lens), max(ctx_lens), Hkv,
                                  128**-0.5, attention.AttentionWorkspace("cuda"), nsplit=nsplit,
                                  split_tokens=split_tokens)
        for _ in range(2):  # the same call again: the scratch now holds this very shape's leftovers
            out = torch.zeros_like(q)
            before = torch.cuda.memory_allocated()
            rc = _call_noalloc(lib, out, pool, tables, q, q_start, ctx, q_lens, Hq, Hkv, nsplit, split_tokens)
            torch.cuda.synchronize()
            assert rc == 0
            assert torch.cuda.memory_allocated() == before  # torch's allocator was not touched by the call
            err = (out.float() - ref.float()).abs().max().item()
            assert err < 3e-2, err
        assert ref.float().abs().max().item() > 0.01  # the comparison is not vacuous


def test_noalloc_entry_rejects_oversized_requests():
    from daser_b200.ops import _lib

    lib = _lib.lib()
    pool, tables, q, q_start, ctx = _case(13, [1], [64], 8, 1)
    out = torch.full_like(q, 7.0)
    pool_c = pool.c_struct()
    # total_q * Hq * nsplit = 1 * 8 * 4096 > 16384 entries of scratch
    rc = lib.daser_paged_attention_fp8_noalloc(
        C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()), C.byref(pool_c), 0, 0,
        C.c_void_p(tables.data_ptr()), int(tables.shape[1]), C.c_void_p(q_start.data_ptr()),
        C.c_void_p(ctx.data_ptr()), 1, 1, 1, 8, 1, 128, 16, 4096, 16, C.c_float(0.088),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == -3
    assert torch.equal(out, torch.full_like(q, 7.0))  # nothing was launched
