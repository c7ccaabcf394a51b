"""fp8 paged attention against fp32 attention over the dequantised cache."""

import pytest
import torch

from daser_b200.kv import codec

pytestmark = pytest.mark.gpu


def _build(num_seqs, q_lens, ctx_lens, Hq, Hkv, n_blocks, seed=0):
    from daser_b200.ops import kv_ops

    torch.manual_seed(seed)
    D, B, L = 128, 16, 2
    kv = torch.randn(L, n_blocks, 2, Hkv, B, D) * 1.0
    payload, scales = codec.quantize_fp8b16(kv)
    deq = codec.dequantize_fp8b16(payload, scales)  # what the kernel sees
    pool = kv_ops.PagedKVPool.from_tensors([payload.cuda()], [scales.cuda()], "LNKHTD")
    max_blocks = max(-(-c // B) for c in ctx_lens) + 1
    perm = torch.randperm(n_blocks)
    tables = torch.zeros(num_seqs, max_blocks, dtype=torch.int32)
    used = 0
    for s in range(num_seqs):
        nb = -(-ctx_lens[s] // B)
        tables[s, :nb] = perm[used : used + nb].to(torch.int32)
        used += nb
    Tq = sum(q_lens)
    q = torch.randn(Tq, Hq, D)
    return pool, deq, tables, q


def _reference(deq, layer, tables, q, q_lens, ctx_lens, Hq, Hkv, scale):
    D, B = 128, 16
    outs = []
    qs = 0
    for s, (ql, ctx) in enumerate(zip(q_lens, ctx_lens)):
        nb = -(-ctx // B)
        blk = deq[layer, tables[s, :nb].long()]  # [nb, 2, H, B, D]
        kvs = blk.permute(1, 0, 3, 2, 4).reshape(2, nb * B, Hkv, D)[:, :ctx]
        k = kvs[0].repeat_interleave(Hq // Hkv, dim=1)
        v = kvs[1].repeat_interleave(Hq // Hkv, dim=1)
        qq = q[qs : qs + ql].to(torch.bfloat16).float()
        sc = torch.einsum("thd,shd->hts", qq, k) * scale
        key = torch.arange(ctx)
        lim = (ctx - ql + torch.arange(ql))[:, None]
        sc = sc.masked_fill((key[None, :] > lim)[None], float("-inf"))
        outs.append(torch.einsum("hts,shd->thd", sc.softmax(-1), v))
        qs += ql
    return torch.cat(outs)


@pytest.mark.parametrize(
    "q_lens,ctx_lens,Hq,Hkv,split",
    [
        ([1], [16], 8, 1, None),
        ([1, 1, 1], [100, 33, 512], 8, 1, None),
        ([1, 1], [700, 1500], 64, 8, None),       # decode, GQA 8:1, several KV heads
        ([1, 1], [700, 1500], 64, 8, (4, 384)),   # forced split-KV
        ([5], [37], 8, 2, None),                    # G = 4
        ([64], [2112], 16, 2, None),                # chunked prefill tail over a long context
        ([7, 1, 20], [39, 300, 20], 8, 1, (2, 160)),  # ragged batch, pure prefill of seq 2
    ],
)
def test_paged_attention_matches_reference(q_lens, ctx_lens, Hq, Hkv, split):
    from daser_b200.ops import attention

    num_seqs = len(q_lens)
    n_blocks = sum(-(-c // 16) for c in ctx_lens) + 4
    pool, deq, tables, q = _build(num_seqs, q_lens, ctx_lens, Hq, Hkv, n_blocks)
    scale = 128**-0.5
    layer = 1
    qd = q.to(torch.bfloat16).cuda()
    out = torch.zeros_like(qd)
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ws = attention.AttentionWorkspace("cuda")
    kw = {}
    if split:
        kw = dict(nsplit=split[0], split_tokens=split[1])
    attention.paged_attention(qd, out, pool, layer, tables.cuda(), q_start,
                              torch.tensor(ctx_lens, dtype=torch.int32, device="cuda"), max(q_lens),
                              max(ctx_lens), Hkv, scale, ws, **kw)
    torch.cuda.synchronize()
    ref = _reference(deq, layer, tables, q, q_lens, ctx_lens, Hq, Hkv, scale)
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 3e-2, err


def _run(q_lens, ctx_lens, Hq, Hkv, split=None, seed=0):
    from daser_b200.ops import attention

    num_seqs = len(q_lens)
    n_blocks = sum(-(-c // 16) for c in ctx_lens) + 4
    pool, deq, tables, q = _build(num_seqs, q_lens, ctx_lens, Hq, Hkv, n_blocks, seed)
    scale = 128**-0.5
    qd = q.to(torch.bfloat16).cuda()
    out = torch.zeros_like(qd)
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ws = attention.AttentionWorkspace("cuda")
    kw = dict(nsplit=split[0], split_tokens=split[1]) if split else {}
    attention.paged_attention(qd, out, pool, 1, tables.cuda(), q_start,
                              torch.tensor(ctx_lens, dtype=torch.int32, device="cuda"), max(q_lens),
                              max(ctx_lens), Hkv, scale, ws, **kw)
    torch.cuda.synchronize()
    ref = _reference(deq, 1, tables, q, q_lens, ctx_lens, Hq, Hkv, scale)
    return out.float().cpu(), ref


@pytest.mark.parametrize(
    "q_lens,ctx_lens,Hq,Hkv,split",
    [
        ([64], [3328], 64, 8, None),              # the RAG query step: 64 new tokens over restored chunks
        ([64], [3261], 8, 1, None),               # one KV head per rank (TP = 8), ragged context end
        ([16], [16], 8, 1, None),                 # a single tile, causal inside it
        ([100], [100], 16, 2, None),              # pure prefill: whole tiles masked for early rows
        ([48, 80], [1000, 81], 32, 8, None),      # G = 4, two sequences, the second barely longer than its query
        ([70], [700], 32, 2, (3, 240)),           # G = 16; split length not a multiple of the key tile
        ([130], [513], 4, 4, (1, 576)),           # G = 1, one split, three row groups
    ],
)
def test_tensor_core_prefill_matches_reference_and_mma_path(q_lens, ctx_lens, Hq, Hkv, split):
    from daser_b200.ops import attention

    try:
        attention.set_tensor_core_prefill(True)
        out_tc, ref = _run(q_lens, ctx_lens, Hq, Hkv, split)
        assert attention.tc_status() == 0
        attention.set_tensor_core_prefill(False)
        out_mma, _ = _run(q_lens, ctx_lens, Hq, Hkv, split)
    finally:
        attention.set_tensor_core_prefill(True)
    assert (out_tc - ref).abs().max().item() < 3e-2
    assert (out_mma - ref).abs().max().item() < 3e-2
    assert (out_tc - out_mma).abs().max().item() < 2e-2
    assert torch.isfinite(out_tc).all()


def test_tensor_core_prefill_ignores_garbage_beyond_the_context():
    """Pages past the context end hold NaN patterns (0x7f payload, NaN scales): masked keys must
    not leak into the output through 0 x NaN."""
    from daser_b200.ops import attention, kv_ops

    torch.manual_seed(4)
    D, B, Hkv, Hq, ctx, ql = 128, 16, 1, 8, 200, 32
    nb = 16
    kv = torch.randn(1, nb, 2, Hkv, B, D)
    payload, scales = codec.quantize_fp8b16(kv)
    deq = codec.dequantize_fp8b16(payload, scales)
    tables = torch.arange(nb, dtype=torch.int32)[None]
    payload[0, 12:, :, :, 8:] = 0x7F   # tokens 200.. of block 12 onwards: e4m3 NaN
    payload[0, 13:] = 0x7F
    scales[0, 13:] = float("nan")
    pool = kv_ops.PagedKVPool.from_tensors([payload.cuda()], [scales.cuda()], "LNKHTD")
    q = torch.randn(ql, Hq, D)
    qd = q.to(torch.bfloat16).cuda()
    out = torch.zeros_like(qd)
    ws = attention.AttentionWorkspace("cuda")
    attention.paged_attention(qd, out, pool, 0, tables.cuda(), torch.tensor([0, ql], dtype=torch.int32, device="cuda"),
                              torch.tensor([ctx], dtype=torch.int32, device="cuda"), ql, ctx, Hkv, D**-0.5, ws)
    torch.cuda.synchronize()
    ref = _reference(deq, 0, tables, q, [ql], [ctx], Hq, Hkv, D**-0.5)
    assert torch.isfinite(out).all()
    assert (out.float().cpu() - ref).abs().max().item() < 3e-2
