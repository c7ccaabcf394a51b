import pytest

from daser_b200.config import DaserConfig, geometry_mismatch
from daser_b200.hashing import hash_tokens, prefix_digests


def test_explicit_slot_size_wins():
    assert DaserConfig(slot_size=1024, num_kv_heads=8).resolved_slot_size() == 1024


def test_derived_slot_size_raw():
    cfg = DaserConfig(num_kv_heads=8, head_dim=128, num_layers=28, block_tokens=16, dtype_bytes=2)
    assert cfg.resolved_slot_size() == 8 * 128 * 2 * 28 * 16 * 2
    assert cfg.layer_size() == 8 * 128 * 2 * 16 * 2


def test_llama70b_slot_sizes_match_the_design_numbers():
    raw = DaserConfig(num_kv_heads=8, head_dim=128, num_layers=80)
    fp8 = DaserConfig(num_kv_heads=8, head_dim=128, num_layers=80, codec="fp8b16")
    assert raw.resolved_slot_size() == 5_242_880
    assert fp8.resolved_slot_size() == 3_276_800


@pytest.mark.parametrize("missing", ["num_kv_heads", "head_dim", "num_layers"])
def test_missing_param_is_named(missing):
    kw = dict(num_kv_heads=8, head_dim=128, num_layers=4)
    kw[missing] = 0
    with pytest.raises(ValueError, match=missing):
        DaserConfig(**kw).resolved_slot_size()


def test_geometry_mismatch_ignores_unset_fields():
    a = DaserConfig(slot_size=4096, num_layers=2).geometry()
    b = dict(a, num_layers=0)
    assert geometry_mismatch(a, b) == []
    assert geometry_mismatch(a, dict(a, slot_size=8192))


def test_hash_is_xxh3_128_of_le_int32():
    import struct

    import xxhash

    toks = [1, 2, 70000, 31999]
    assert hash_tokens(toks) == xxhash.xxh3_128(struct.pack("<4i", *toks)).hexdigest()
    assert len(hash_tokens(toks)) == 32


def test_prefix_digests_equal_from_scratch_hashes():
    toks = list(range(100, 100 + 75))
    digs = prefix_digests(toks, 16)
    assert len(digs) == 4
    for i, d in enumerate(digs):
        assert d == hash_tokens(toks[: (i + 1) * 16])
    assert prefix_digests(toks[:5], 16) == []
