import asyncio

import pytest

from daser_b200.hashing import hash_tokens
from daser_b200.position import FixedOffsetEncoder, RopeReencoder, inv_freq_table
from daser_b200.retrieval import ChunkOffsetIndex, PrefixHashIndex
from daser_b200.server.__main__ import _build_daser_config, _parse_args
from daser_b200.server.doc_registry import DocEntry, DocRegistry
from daser_b200.server.metadata_store import ChunkMeta


def cm(tokens, model="m", start=0):
    return ChunkMeta(hash_tokens(tokens), start, -(-len(tokens) // 16), len(tokens), 0, model)


def run(coro):
    return asyncio.run(coro)


def test_prefix_exact_longer_miss_remove_model():
    idx = PrefixHashIndex(16)
    t = list(range(64))
    run(idx.insert(cm(t[:32])))
    assert run(idx.lookup(t[:32], "m"))[0].token_count == 32
    assert run(idx.lookup(t, "m"))[0].token_count == 32  # longer query finds stored prefix
    assert run(idx.lookup(list(range(1, 65)), "m")) == []
    assert run(idx.lookup(t, "other")) == []
    run(idx.insert(cm(t[:48])))
    assert run(idx.lookup(t, "m"))[0].token_count == 48  # longest wins
    run(idx.remove(hash_tokens(t[:48])))
    run(idx.remove("unknown"))
    assert run(idx.lookup(t, "m"))[0].token_count == 32


def test_chunk_offset_scan_finds_aligned_chunks():
    idx = ChunkOffsetIndex(16)
    a, b = list(range(1000, 1048)), list(range(2000, 2020))  # 48 and 20 tokens
    for toks in (a, b):
        run(idx.insert(cm(toks)))
        idx.register_anchor(hash_tokens(toks), hash_tokens(toks[:16]))
    prompt = [7] * 16 + a + b + [0] * 12 + [8] * 16  # b padded to 32
    hits = idx.scan(prompt, "m")
    assert [(h.meta.token_count, h.offset) for h in hits] == [(48, 16), (20, 64)]
    assert idx.scan([7] * 8 + a, "m") == []  # not block aligned
    idx.discard(hash_tokens(a))
    assert [h.offset for h in idx.scan(prompt, "m")] == [64]
    assert idx.lookup_keys([hash_tokens(b), "x"], "m")[1] is None


def test_fixed_offset():
    assert FixedOffsetEncoder().assign_offset("k", 10) == 0
    assert FixedOffsetEncoder(7).assign_offset("k", 10) == 7
    assert FixedOffsetEncoder(7).get_offset(ChunkMeta("k", 0, 1, 16, 42, "m")) == 42


def test_rope_reencoder_delta_and_llama3_scaling():
    pe = RopeReencoder(head_dim=64)
    meta = ChunkMeta("k", 0, 1, 16, pe.assign_offset("k", 16), "m")
    assert pe.delta(meta, 300) == 300
    assert pe.delta(128, 100) == -28
    plain = inv_freq_table(128, 500000.0)
    scaled = inv_freq_table(128, 500000.0, {"factor": 8.0, "low_freq_factor": 1.0,
                                            "high_freq_factor": 4.0,
                                            "original_max_position_embeddings": 8192})
    assert plain[0] == scaled[0] == 1.0
    assert scaled[-1] == pytest.approx(plain[-1] / 8.0)


def test_doc_registry_transitions():
    r = DocRegistry()
    r.insert(DocEntry("d", "t", chunk_keys=["a", "b"]))
    assert r.get("d").cached_mask == [True, True]
    with pytest.raises(ValueError):
        r.insert(DocEntry("d", "t"))
    r.mark_chunk_evicted("d", "a")
    assert r.get("d").status == "ready"  # as the reference: ready until the last chunk goes
    r.mark_chunk_evicted("d", "b")
    assert r.get("d").status == "evicted"
    r.mark_chunk_evicted("nope", "a")
    r2 = DocRegistry()
    r2.load_dict(r.to_dict())
    assert r2.get("d").cached_mask == [False, False] and len(r2) == 1
    assert r.remove("d").doc_id == "d" and r.remove("d") is None


def test_cli_defaults_and_validation():
    cfg = _build_daser_config(_parse_args(["--store-path", "/x/daser.store"]))
    assert cfg.total_slots == 5120 and cfg.slot_size == 2 * 1024 * 1024
    assert cfg.ipc_socket_path == "/tmp/daser.sock" and cfg.index_path == "/tmp/daser.index"
    with pytest.raises(ValueError, match="multiple"):
        _build_daser_config(_parse_args(["--store-path", "/x", "--store-size", "1000001"]))
    with pytest.raises(SystemExit):
        _parse_args([])
    cfg = _build_daser_config(_parse_args([
        "--store-path", "/x", "--slot-size", "0", "--num-kv-heads", "8", "--head-dim", "128",
        "--num-layers", "32", "--store-size", str(2097152 * 10)]))
    assert cfg.slot_size == 0 and cfg.resolved_slot_size() == 2097152 and cfg.total_slots == 10  # kept unresolved, as the reference does
