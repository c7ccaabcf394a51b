import pytest
import torch

from daser_b200.config import DaserConfig
from daser_b200.kv import codec
from daser_b200.kv.layout import KVGeometry, owner_rank, tp_head_range
from daser_b200.position import inv_freq_table


def test_geometry_matches_config_slot_size():
    for c in ("raw", "fp8b16"):
        cfg = DaserConfig(num_kv_heads=8, head_dim=128, num_layers=80, codec=c)
        geo = KVGeometry.from_config(cfg)
        assert geo.slot_size == cfg.resolved_slot_size()
        assert geo.layer_offset(3, 2, 5) == 5 * geo.slot_size + 5 * geo.layer_size


def test_tp_head_ranges():
    assert tp_head_range(8, 1, 0) == (0, 8)
    assert tp_head_range(8, 4, 3) == (6, 2)
    assert tp_head_range(8, 8, 5) == (5, 1)
    assert tp_head_range(2, 8, 5) == (1, 1)  # replicated heads
    with pytest.raises(ValueError):
        tp_head_range(8, 3, 0)
    assert 0 <= owner_rank("00ff" * 8, 8) < 8 and owner_rank("ab" * 16, 1) == 0


def test_fp8_roundtrip_error_bound():
    torch.manual_seed(0)
    x = torch.randn(64, 8, 128) * 0.5
    q, s = codec.quantize_fp8b16(x)
    assert q.dtype == torch.uint8 and s.shape == (64, 8, 8)
    y = codec.dequantize_fp8b16(q, s)
    # e4m3 has 3 mantissa bits: relative step 2^-3, half of it after rounding,
    # measured against the group's absmax for the small elements
    gmax = x.reshape(64, 8, 8, 16).abs().amax(-1, keepdim=True).expand(-1, -1, -1, 16).reshape_as(x)
    assert ((y - x).abs() <= gmax * 2**-4 + 1e-12).all()
    # the group maximum survives up to fp32 rounding of the scale
    assert torch.allclose(
        y.abs().reshape(64, 8, 8, 16).amax(-1), x.abs().reshape(64, 8, 8, 16).amax(-1), rtol=1e-6, atol=0
    )


def test_fp8_zero_group_and_bf16_input():
    x = torch.zeros(2, 32, dtype=torch.bfloat16)
    x[1, 3] = 2.0
    q, s = codec.quantize_fp8b16(x)
    assert s[0, 0] == 1.0 and s[0, 1] == 1.0 and s[1, 1] == 1.0
    y = codec.dequantize_fp8b16(q, s, torch.bfloat16)
    assert torch.equal(y, x)


def test_rope_delta_composes():
    torch.manual_seed(1)
    inv = inv_freq_table(64, 10000.0)
    x = torch.randn(5, 3, 64)
    pos = torch.arange(5)
    c0, s0 = codec.rope_cos_sin(pos, inv)
    c1, s1 = codec.rope_cos_sin(pos + 37, inv)
    at0 = codec.rope_rotate(x, c0, s0)
    at37 = codec.rope_rotate(x, c1, s1)
    moved = codec.rope_delta_rotate(at0, 37, inv)
    assert torch.allclose(moved, at37, atol=1e-5)
    assert torch.equal(codec.rope_delta_rotate(at0, 0, inv), at0)


@pytest.mark.parametrize("c", ["raw", "fp8b16"])
def test_pack_unpack_layer(c):
    torch.manual_seed(2)
    geo = KVGeometry(2, 2, 32, 16, 2, c)
    k = (torch.randn(16, 2, 32) * 0.5).to(torch.bfloat16)
    v = (torch.randn(16, 2, 32) * 0.5).to(torch.bfloat16)
    raw = codec.pack_layer(geo, k, v)
    assert raw.numel() == geo.layer_size
    k2, v2 = codec.unpack_layer(geo, raw, torch.float32)
    if c == "raw":
        assert torch.equal(k2, k.float()) and torch.equal(v2, v.float())
        # byte-identical to the reference container: K block then V block
        assert torch.equal(raw[: raw.numel() // 2], k.contiguous().view(torch.uint8).reshape(-1))
    else:
        assert torch.allclose(k2, k.float(), atol=0.2, rtol=0.07)


def test_restore_reference_selects_heads_and_rotates_only_k():
    torch.manual_seed(3)
    geo = KVGeometry(2, 4, 32, 16, 4, "raw")
    ks = [torch.randn(16, 4, 32) for _ in range(2)]
    vs = [torch.randn(16, 4, 32) for _ in range(2)]
    slot = codec.pack_slot(geo, ks, vs)
    assert slot.numel() == geo.slot_size
    inv = inv_freq_table(32)
    out = codec.restore_slot_reference(geo, slot, 11, inv, head_range=(2, 2))
    assert out[1][1].shape == (16, 2, 32)
    assert torch.equal(out[1][1], vs[1][:, 2:4])
    assert torch.allclose(out[0][0], codec.rope_delta_rotate(ks[0], 11, inv)[:, 2:4])
