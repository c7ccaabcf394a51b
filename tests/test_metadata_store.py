import msgpack
import pytest

from daser_b200.server.metadata_store import ChunkMeta, MetadataStore


def meta(key, start, n, toks=None):
    return ChunkMeta(key, start, n, toks or n * 16, 0, "m")


def test_insert_get_len():
    s = MetadataStore(16)
    s.insert(meta("a", 0, 3))
    assert len(s) == 1 and s.get("a").num_slots == 3 and s.get("zz") is None


def test_slot_map_kinds():
    s = MetadataStore(16)
    s.insert(meta("a", 2, 3))
    assert s.get_slot_entry(2).kind == "chunk" and s.get_slot_entry(2).chunk_key == "a"
    assert s.get_slot_entry(3).kind == "cont" and s.get_slot_entry(4).kind == "cont"
    with pytest.raises(IndexError):
        s.get_slot_entry(16)


def test_remove_tombstones_the_run():
    s = MetadataStore(16)
    s.insert(meta("a", 0, 3))
    s.remove("a")
    assert s.get("a") is None and len(s) == 0
    e = s.get_slot_entry(0)
    assert e.kind == "skip" and e.num_slots == 3


def test_remove_missing_raises_keyerror():
    with pytest.raises(KeyError):
        MetadataStore(4).remove("nope")


def test_duplicate_key_raises_valueerror():
    s = MetadataStore(16)
    s.insert(meta("a", 0, 1))
    with pytest.raises(ValueError):
        s.insert(meta("a", 4, 1))


def test_out_of_range_run_rejected():
    with pytest.raises(ValueError):
        MetadataStore(4).insert(meta("a", 3, 2))


def test_insert_skip():
    s = MetadataStore(8)
    s.insert_skip(6, 2)
    assert s.get_slot_entry(6).kind == "skip" and s.get_slot_entry(6).num_slots == 2
    assert s.get_slot_entry(7).kind == "cont"


def test_save_load_roundtrip_and_reference_shape(tmp_path):
    s = MetadataStore(8)
    s.insert(meta("a", 0, 3))
    s.insert_skip(6, 2)
    p = str(tmp_path / "i.msgpack")
    s.save(p)
    raw = msgpack.unpackb(open(p, "rb").read(), raw=False)
    # the reference's payload: three keys, one slot_map entry per slot
    assert set(raw) == {"total_slots", "chunk_index", "slot_map"}
    assert len(raw["slot_map"]) == 8
    assert set(raw["slot_map"][0]) == {"kind", "chunk_key", "num_slots"}
    assert set(raw["chunk_index"]["a"]) == {
        "chunk_key", "start_slot", "num_slots", "token_count", "pos_offset",
        "model_id", "created_at", "doc_ids",
    }
    t = MetadataStore(8)
    t.load(p)
    assert t.get("a").start_slot == 0 and t.get_slot_entry(6).kind == "skip"


def test_load_demotes_dangling_chunk_heads():
    # a snapshot written after the reference's non-tombstoning remove()
    payload = {
        "total_slots": 4,
        "chunk_index": {},
        "slot_map": [{"kind": "chunk", "chunk_key": "gone", "num_slots": 2}]
        + [{"kind": "cont", "chunk_key": None, "num_slots": 0}] * 3,
    }
    s = MetadataStore(4)
    s.from_bytes(msgpack.packb(payload, use_bin_type=True))
    assert s.get_slot_entry(0).kind == "skip"


def test_commit_state_side_table():
    s = MetadataStore(8)
    s.insert(meta("a", 0, 1), committed=False)
    assert not s.is_committed("a")
    s.mark_committed("a", checksum=123)
    assert s.is_committed("a") and s.checksum("a") == 123
