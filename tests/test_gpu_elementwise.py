import pytest
import torch

from daser_b200.kv import codec
from daser_b200.position import inv_freq_table

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hidden", [256, 4096, 8192])
@pytest.mark.parametrize("fp32_in", [False, True])
def test_add_rmsnorm(hidden, fp32_in):
    from daser_b200.ops import elementwise as ew

    torch.manual_seed(0)
    T = 7
    x = torch.randn(T, hidden, device="cuda")
    xin = x.clone() if fp32_in else x.to(torch.bfloat16)
    res = torch.randn(T, hidden, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    res_ref = (xin.float() + res.float()).to(torch.bfloat16)
    h = res_ref.float()
    ref = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    res_io = res.clone()
    out = ew.add_rmsnorm(xin, w, residual=res_io, zero_after=fp32_in)
    torch.cuda.synchronize()
    assert torch.equal(res_io, res_ref)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    if fp32_in:
        assert xin.abs().max().item() == 0  # accumulator handed back zeroed
    out2 = ew.add_rmsnorm(x.to(torch.bfloat16), w)  # no residual
    h2 = x.to(torch.bfloat16).float()
    ref2 = h2 * torch.rsqrt(h2.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert torch.allclose(out2.float(), ref2, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("pool_fp8", [False, True])
@pytest.mark.parametrize("fp32_in", [False, True])
def test_rope_kv_write(pool_fp8, fp32_in):
    from daser_b200.ops import elementwise as ew
    from daser_b200.ops import kv_ops

    torch.manual_seed(1)
    T, Hq, Hkv, D, B, L, NB = 9, 4, 2, 64, 16, 2, 5
    inv = inv_freq_table(D, 10000.0)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda")
    qkv_in = qkv.clone() if fp32_in else qkv.to(torch.bfloat16)
    src = qkv_in.float().cpu()
    positions = torch.tensor([0, 1, 2, 40, 41, 42, 100, 7, 300], dtype=torch.int32, device="cuda")
    slots = torch.tensor([0, 1, 2, 16, 17, 18, 79, -1, 33], dtype=torch.int64, device="cuda")
    if pool_fp8:
        payload = torch.zeros(L, NB, 2, Hkv, B, D, dtype=torch.uint8, device="cuda")
        scales = torch.zeros(L, NB, 2, Hkv, B, D // 16, dtype=torch.float32, device="cuda")
        pool = kv_ops.PagedKVPool.from_tensors([payload], [scales], "LNKHTD")
    else:
        payload = torch.zeros(L, NB, 2, Hkv, B, D, dtype=torch.bfloat16, device="cuda")
        pool = kv_ops.PagedKVPool.from_tensors([payload], None, "LNKHTD")
    cos_sin = kv_ops.rope_table(512, inv, "cuda")
    q_out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device="cuda")
    ew.rope_kv_write(qkv_in, positions, slots, cos_sin, q_out, Hq, Hkv, D, B, pool, layer=1, zero_after=fp32_in)
    torch.cuda.synchronize()
    cos, sin = codec.rope_cos_sin(positions.cpu(), inv)
    q = src[:, : Hq * D].reshape(T, Hq, D)
    k = src[:, Hq * D : (Hq + Hkv) * D].reshape(T, Hkv, D)
    v = src[:, (Hq + Hkv) * D :].reshape(T, Hkv, D)
    q_ref, k_ref = codec.rope_rotate(q, cos, sin), codec.rope_rotate(k, cos, sin)
    assert torch.allclose(q_out.float().cpu(), q_ref, atol=2e-2, rtol=2e-2)
    if pool_fp8:
        cache = codec.dequantize_fp8b16(payload.cpu(), scales.cpu())
        tol = dict(atol=0.15, rtol=0.13)
    else:
        cache = payload.float().cpu()
        tol = dict(atol=2e-2, rtol=2e-2)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        blk, off = divmod(s, B)
        assert torch.allclose(cache[1, blk, 0, :, off], k_ref[t], **tol)
        assert torch.allclose(cache[1, blk, 1, :, off], v[t].to(torch.bfloat16).float(), **tol)
    assert cache[0].abs().max() == 0
    if fp32_in:
        assert qkv_in.abs().max().item() == 0


def test_swiglu_embedding_argmax():
    from daser_b200.ops import elementwise as ew

    torch.manual_seed(2)
    x = torch.randn(5, 2 * 256, device="cuda")
    y = ew.swiglu(x.to(torch.bfloat16))
    xb = x.to(torch.bfloat16).float()
    ref = torch.nn.functional.silu(xb[:, :256]) * xb[:, 256:]
    assert torch.allclose(y.float(), ref, atol=2e-2, rtol=2e-2)
    acc = x.clone()
    y2 = ew.swiglu(acc, zero_after=True)
    assert torch.allclose(y2.float(), torch.nn.functional.silu(x[:, :256]) * x[:, 256:], atol=2e-2, rtol=2e-2)
    assert acc.abs().max().item() == 0
    table = torch.randn(100, 64, device="cuda").to(torch.bfloat16)
    ids = torch.tensor([3, 99, 0, 50], dtype=torch.int32, device="cuda")
    assert torch.equal(ew.embedding(ids, table), table[ids.long()])
    # vocab-parallel shard: ids outside [begin, begin + rows) give zeros
    part = ew.embedding(ids, table[40:60].contiguous(), vocab_begin=40)
    assert torch.equal(part[3], table[50]) and part[0].abs().max() == 0
    logits = torch.randn(3, 1024, device="cuda")
    logits[1, 777] = 50.0
    bv = torch.empty(3, device="cuda")
    bi = torch.empty(3, dtype=torch.int32, device="cuda")
    ew.argmax(logits, bv, bi, index_offset=1000)
    assert bi.tolist() == [int(i) + 1000 for i in logits.argmax(-1)]
    assert torch.equal(bv, logits.max(-1).values)
