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
