"""CUDA codec / restore / save kernels against the fp32 CPU oracle in ``kv/codec.py``."""

import pytest
import torch

from daser_b200.kv import codec
from daser_b200.kv.layout import KVGeometry, tp_head_range
from daser_b200.position import inv_freq_table

pytestmark = pytest.mark.gpu


def _ops():
    from daser_b200.ops import kv_ops

    return kv_ops


def test_quant_matches_oracle_bitwise():
    kv_ops = _ops()
    torch.manual_seed(0)
    x = (torch.randn(37, 8, 128) * 0.5).to(torch.bfloat16)
    x[3, 2, 16:32] = 0  # an all-zero group
    q_ref, s_ref = codec.quantize_fp8b16(x)
    q, s = kv_ops.quantize_fp8b16(x.cuda())
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref)
    y = kv_ops.dequantize_fp8b16(q, s)
    y_ref = codec.dequantize_fp8b16(q_ref, s_ref, torch.bfloat16)
    assert torch.equal(y.cpu(), y_ref)


def _make_pool(geo, n_blocks, tp, fp8, layout, device="cuda"):
    """Per-rank pools (all on one device: the ranks are emulated by one kernel)."""
    h0, hn = tp_head_range(geo.num_kv_heads, tp, 0)
    dims = {"L": geo.num_layers, "N": n_blocks, "K": 2, "T": geo.block_tokens, "H": hn, "D": geo.head_dim}
    shape = [dims[c] for c in layout]
    payloads, scales = [], []
    for _ in range(tp):
        if fp8:
            payloads.append(torch.zeros(shape, dtype=torch.uint8, device=device))
            scales.append(torch.zeros(shape[:-1] + [geo.head_dim // 16], dtype=torch.float32, device=device))
        else:
            payloads.append(torch.zeros(shape, dtype=torch.bfloat16, device=device))
    return payloads, (scales if fp8 else None)


def _pool_block(payloads, scales, layout, rank, layer, block, fp8):
    """(k, v) float32 [T, H, D] of one block of one rank, whatever the layout."""
    t = payloads[rank]
    perm = [layout.index(c) for c in "LNKTHD"]
    x = t.permute(perm)[layer, block]  # [K, T, H, D]
    if fp8:
        s = scales[rank].permute(perm)[layer, block]
        x = codec.dequantize_fp8b16(x.contiguous().cpu(), s.contiguous().cpu())
    else:
        x = x.float().cpu()
    return x[0], x[1]


@pytest.mark.parametrize("img_codec", ["fp8b16", "raw"])
@pytest.mark.parametrize("pool_fp8", [False, True])
@pytest.mark.parametrize("tp,layout", [(1, "LNKHTD"), (4, "LNKHTD"), (2, "LKNTHD")])
def test_restore_matches_oracle(img_codec, pool_fp8, tp, layout):
    kv_ops = _ops()
    torch.manual_seed(1)
    geo = KVGeometry(num_layers=3, num_kv_heads=4, head_dim=64, block_tokens=16, dtype_bytes=2, codec=img_codec)
    inv = inv_freq_table(64, 10000.0)
    n_slots, n_blocks = 5, 11
    slots = []
    for _ in range(n_slots):
        ks = [(torch.randn(16, 4, 64) * 0.5).to(torch.bfloat16) for _ in range(3)]
        vs = [(torch.randn(16, 4, 64) * 0.5).to(torch.bfloat16) for _ in range(3)]
        slots.append(codec.pack_slot(geo, ks, vs))
    staging = torch.stack(slots).cuda()
    blocks = [7, 0, 10, 3, 5]
    deltas = [0, 17, -5, 300, 1]
    work = kv_ops.KVWorkList(
        slot_ptrs=torch.tensor([staging.data_ptr() + i * geo.slot_size for i in range(n_slots)], dtype=torch.int64, device="cuda"),
        block_ids=torch.tensor(blocks, dtype=torch.int32, device="cuda"),
        deltas=torch.tensor(deltas, dtype=torch.int32, device="cuda"),
    )
    payloads, scales = _make_pool(geo, n_blocks, tp, pool_fp8, layout)
    pool = kv_ops.PagedKVPool.from_tensors(payloads, scales, layout)
    cos_sin = kv_ops.rope_table(512, inv, "cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    kv_ops.kv_restore(work, geo, pool, cos_sin, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]
    for i in range(n_slots):
        for rank in range(tp):
            ref = codec.restore_slot_reference(geo, slots[i], deltas[i], inv, tp_head_range(4, tp, rank))
            for layer in range(3):
                k, v = _pool_block(payloads, scales, layout, rank, layer, blocks[i], pool_fp8)
                k_ref, v_ref = ref[layer]
                if pool_fp8:
                    # one more fp8 rounding on top of the oracle's fp32 values
                    k_q = codec.dequantize_fp8b16(*codec.quantize_fp8b16(k_ref))
                    v_q = codec.dequantize_fp8b16(*codec.quantize_fp8b16(v_ref))
                    assert torch.allclose(k, k_q, atol=2e-2, rtol=7e-2)
                    assert torch.allclose(v, v_q, atol=1e-6, rtol=0) or torch.allclose(v, v_q, atol=2e-2, rtol=7e-2)
                else:
                    assert torch.allclose(k, k_ref.to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)
                    assert torch.equal(v, v_ref.to(torch.bfloat16).float())
    # untouched blocks stay zero
    k, v = _pool_block(payloads, scales, layout, 0, 0, 1, pool_fp8)
    assert k.abs().max() == 0


def test_restore_reports_bad_block_instead_of_faulting():
    kv_ops = _ops()
    geo = KVGeometry(1, 2, 32, 16, 2, "raw")
    staging = torch.zeros(geo.slot_size, dtype=torch.uint8, device="cuda")
    payloads, _ = _make_pool(geo, 4, 1, False, "LNKHTD")
    pool = kv_ops.PagedKVPool.from_tensors(payloads, None, "LNKHTD")
    work = kv_ops.KVWorkList(
        torch.tensor([staging.data_ptr()], dtype=torch.int64, device="cuda"),
        torch.tensor([99], dtype=torch.int32, device="cuda"),
    )
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    kv_ops.kv_restore(work, geo, pool, None, status)
    torch.cuda.synchronize()
    assert status.tolist() == [2, 0]


@pytest.mark.parametrize("img_codec", ["fp8b16", "raw"])
@pytest.mark.parametrize("pool_fp8", [False, True])
@pytest.mark.parametrize("tp", [1, 2])
def test_save_then_restore_roundtrip(img_codec, pool_fp8, tp):
    kv_ops = _ops()
    torch.manual_seed(2)
    geo = KVGeometry(2, 4, 64, 16, 2, img_codec)
    n_blocks = 6
    payloads, scales = _make_pool(geo, n_blocks, tp, pool_fp8, "LNKHTD")
    # fill every rank's pool with data
    truth = (torch.randn(2, n_blocks, 2, 4, 16, 64) * 0.5).to(torch.bfloat16)  # [L, N, K, H, T, D] all heads
    hn = 4 // tp
    for r in range(tp):
        part = truth[:, :, :, r * hn : (r + 1) * hn].contiguous().cuda()
        if pool_fp8:
            q, s = kv_ops.quantize_fp8b16(part)
            payloads[r].copy_(q)
            scales[r].copy_(s)
        else:
            payloads[r].copy_(part)
    pool = kv_ops.PagedKVPool.from_tensors(payloads, scales, "LNKHTD")
    blocks = [4, 1, 2]
    staging = torch.zeros(len(blocks) * geo.slot_size, dtype=torch.uint8, device="cuda")
    work = kv_ops.KVWorkList(
        torch.tensor([staging.data_ptr() + i * geo.slot_size for i in range(len(blocks))], dtype=torch.int64, device="cuda"),
        torch.tensor(blocks, dtype=torch.int32, device="cuda"),
    )
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    for r in range(tp):  # each rank writes its head slice of the same slot images
        kv_ops.kv_save(work, geo, pool, r, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]
    img = staging.cpu()
    for i, b in enumerate(blocks):
        for layer in range(2):
            raw = img[i * geo.slot_size + layer * geo.layer_size : i * geo.slot_size + (layer + 1) * geo.layer_size]
            k, v = codec.unpack_layer(geo, raw)  # [T, H, D]
            k_true = truth[layer, b, 0].permute(1, 0, 2).float()
            v_true = truth[layer, b, 1].permute(1, 0, 2).float()
            exact = img_codec == "raw" and not pool_fp8
            if exact:
                assert torch.equal(k, k_true) and torch.equal(v, v_true)
            else:
                assert torch.allclose(k, k_true, atol=0.15, rtol=0.13)
                assert torch.allclose(v, v_true, atol=0.15, rtol=0.13)
    # raw image of a bf16 pool is byte-identical to the reference container
    if img_codec == "raw" and not pool_fp8 and tp == 1:
        k0 = truth[0, blocks[0], 0].permute(1, 0, 2).contiguous()
        assert torch.equal(img[: k0.numel() * 2], k0.view(torch.uint8).reshape(-1))


@pytest.mark.parametrize("pool_fp8", [False, True])
def test_restore_and_save_stay_inside_their_buffers(pool_fp8):
    """Guard bytes on both sides of the pool, the scale table and the staging area survive a
    restore into the first and last block and a save of the same blocks."""
    kv_ops = _ops()
    torch.manual_seed(3)
    geo = KVGeometry(2, 2, 64, 16, 2, "fp8b16")
    n_blocks, guard = 5, 4096
    elems = geo.num_layers * n_blocks * 2 * 2 * 16 * 64
    pool_bytes = elems * (1 if pool_fp8 else 2)
    raw_pool = torch.full((guard + pool_bytes + guard,), 0xA5, dtype=torch.uint8, device="cuda")
    raw_scales = torch.full((guard + elems // 16 * 4 + guard,), 0xA5, dtype=torch.uint8, device="cuda")
    shape = [geo.num_layers, n_blocks, 2, 2, 16, 64]
    body = raw_pool[guard : guard + pool_bytes]
    payload = (body if pool_fp8 else body.view(torch.bfloat16)).view(shape)
    scales = raw_scales[guard:-guard].view(torch.float32).view(shape[:-1] + [4]) if pool_fp8 else None
    pool = kv_ops.PagedKVPool.from_tensors([payload], [scales] if pool_fp8 else None, "LNKHTD")
    n = 2
    raw_staging = torch.full((guard + n * geo.slot_size + guard,), 0xA5, dtype=torch.uint8, device="cuda")
    ks = [(torch.randn(16, 2, 64) * 0.5).to(torch.bfloat16) for _ in range(2)]
    vs = [(torch.randn(16, 2, 64) * 0.5).to(torch.bfloat16) for _ in range(2)]
    image = codec.pack_slot(geo, ks, vs).cuda()
    for i in range(n):
        raw_staging[guard + i * geo.slot_size : guard + (i + 1) * geo.slot_size] = image
    ptrs = torch.tensor([raw_staging.data_ptr() + guard + i * geo.slot_size for i in range(n)], dtype=torch.int64,
                        device="cuda")
    work = kv_ops.KVWorkList(ptrs, torch.tensor([0, n_blocks - 1], dtype=torch.int32, device="cuda"),
                             torch.tensor([3, -7], dtype=torch.int32, device="cuda"))
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    kv_ops.kv_restore(work, geo, pool, kv_ops.rope_table(64, inv_freq_table(64, 10000.0), "cuda"), status)
    kv_ops.kv_save(kv_ops.KVWorkList(ptrs, work.block_ids), geo, pool, 0, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]
    for buf in (raw_pool, raw_scales, raw_staging):
        assert bool((buf[:guard] == 0xA5).all()) and bool((buf[-guard:] == 0xA5).all())
    assert bool((payload.view(torch.uint8) != 0xA5).any())  # the kernels did write


def test_restore_by_layer_groups_equals_one_launch():
    """The pipelined restore launches the kernel once per group of layers: together the pieces
    write exactly what one launch over all layers writes, and a piece touches no other layer."""
    kv_ops = _ops()
    torch.manual_seed(4)
    geo = KVGeometry(num_layers=6, num_kv_heads=8, head_dim=128, block_tokens=16, dtype_bytes=2, codec="fp8b16")
    n_slots, n_blocks = 7, 16
    staging = torch.randint(0, 256, (n_slots, geo.slot_size), dtype=torch.uint8)
    # plausible scales (the payload bytes may be anything but NaN patterns: keep exponents small)
    per_layer = staging.view(n_slots, geo.num_layers, geo.layer_size)
    per_layer[..., : geo.payload_bytes_per_layer] &= 0x77
    sc = torch.rand(n_slots, geo.num_layers, (geo.layer_size - geo.payload_bytes_per_layer) // 4) * 0.01 + 0.001
    per_layer[..., geo.payload_bytes_per_layer :] = sc.view(torch.uint8).view(n_slots, geo.num_layers, -1)
    staging = staging.cuda()
    work = kv_ops.KVWorkList(
        slot_ptrs=torch.tensor([staging.data_ptr() + i * geo.slot_size for i in range(n_slots)], dtype=torch.int64, device="cuda"),
        block_ids=torch.tensor([3, 9, 0, 15, 7, 1, 12], dtype=torch.int32, device="cuda"),
        deltas=torch.tensor([0, 40, 0, -3, 7, 0, 100], dtype=torch.int32, device="cuda"),
    )
    cos_sin = kv_ops.rope_table(256, inv_freq_table(128, 500000.0), "cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    for tp in (1, 2):
        pa, sa = _make_pool(geo, n_blocks, tp, True, "LNKHTD")
        pb, sb = _make_pool(geo, n_blocks, tp, True, "LNKHTD")
        kv_ops.kv_restore(work, geo, kv_ops.PagedKVPool.from_tensors(pa, sa, "LNKHTD"), cos_sin, status)
        pool_b = kv_ops.PagedKVPool.from_tensors(pb, sb, "LNKHTD")
        kv_ops.kv_restore(work, geo, pool_b, cos_sin, status, layer_begin=0, layer_count=1)
        torch.cuda.synchronize()
        assert all(bool((t[1:] == 0).all()) for t in pb)  # only layer 0 so far
        assert all(torch.equal(x[0], y[0]) for x, y in zip(pa, pb))
        kv_ops.kv_restore(work, geo, pool_b, cos_sin, status, layer_begin=1, layer_count=3)
        kv_ops.kv_restore(work, geo, pool_b, cos_sin, status, layer_begin=4, layer_count=0)  # 0 = through the last
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0]
        for x, y in zip(pa + sa, pb + sb):
            assert torch.equal(x, y)
        assert any(bool(t.any()) for t in pa)
    with pytest.raises(Exception):
        kv_ops.kv_restore(work, geo, pool_b, cos_sin, status, layer_begin=5, layer_count=3)


def test_copy_rows_and_flag_signalling():
    from daser_b200.ops import elementwise as ew

    kv_ops = _ops()
    src = torch.arange(8 * 64, dtype=torch.int32).view(torch.uint8).clone().pin_memory()
    dst = torch.zeros(src.numel(), dtype=torch.uint8, device="cuda")
    pitch = src.numel() // 8
    kv_ops.copy_rows(dst.data_ptr() + 16, src.data_ptr() + 16, pitch, 48, 8)  # bytes [16, 64) of each of 8 rows
    torch.cuda.synchronize()
    got, want = dst.cpu().view(8, pitch), src.view(8, pitch)
    assert torch.equal(got[:, 16:64], want[:, 16:64]) and not got[:, :16].any() and not got[:, 64:].any()
    # signal then wait on the same stream: the wait finds the value; a wait for more runs out
    # (bounded) and reports through the status word, and the stream stays usable
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ew.signal_flags([flags.data_ptr() + 4 * i for i in range(3)], 5)
    ew.wait_flags(flags.data_ptr(), 3, 5, status)
    torch.cuda.synchronize()
    assert flags.tolist() == [5, 5, 5, 0, 0, 0, 0, 0] and status[0].item() == 0
