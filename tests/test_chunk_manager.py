import random

import pytest

from daser_b200.server.chunk_manager import ChunkManager, RingInvariantError
from daser_b200.server.doc_registry import DocEntry, DocRegistry
from daser_b200.server.metadata_store import MetadataStore


def make(total=8, docs=None):
    return ChunkManager(total, MetadataStore(total), docs)


def A(m, key, n):
    return m.alloc(key, num_slots=n, token_count=n * 16, model_id="m", pos_offset=0)


def test_first_alloc_starts_at_zero_and_head_advances():
    m = make()
    assert A(m, "k1", 3) == 0
    assert A(m, "k2", 2) == 3
    assert m.head == 5 and m.free_slots == 3


def test_fifo_eviction_when_full():
    m = make(6)
    A(m, "k1", 3), A(m, "k2", 3), A(m, "k3", 3)
    assert m.store.get("k1") is None
    assert m.store.get("k2") is not None and m.store.get("k3") is not None


def test_evict_oldest_advances_tail_and_empty_raises():
    m = make()
    A(m, "k1", 3)
    m.evict_oldest()
    assert m.tail == 3 and m.store.get("k1") is None
    with pytest.raises(RuntimeError):
        m.evict_oldest()


def test_wrap_pads_with_skip_and_restarts_at_zero():
    m = make(8)
    A(m, "k1", 3), A(m, "k2", 3)
    assert A(m, "k3", 4) == 0
    assert m.store.get_slot_entry(6).kind == "skip"
    assert m.store.get("k1") is None and m.store.get("k2") is None


def test_skip_run_is_consumed_after_wrap():
    m = make(8)
    A(m, "k1", 3), A(m, "k2", 3), A(m, "k3", 4)
    assert A(m, "k4", 2) == 4
    A(m, "k5", 2)  # needs the padding at [6,8) reclaimed, then lands there
    assert m.store.get("k5").start_slot == 6


def test_too_large_rejected():
    with pytest.raises(ValueError):
        A(make(4), "k", 5)


def test_duplicate_committed_key_rejected_before_ring_mutation():
    m = make(8)
    A(m, "k1", 3), A(m, "k2", 3)
    head, tail = m.head, m.tail
    with pytest.raises(ValueError):
        A(m, "k1", 4)  # would wrap and evict if the check came late
    assert (m.head, m.tail) == (head, tail) and m.store.get("k2") is not None


def test_uncommitted_realloc_is_idempotent():
    m = make(8)
    s1 = m.alloc("k", 2, 32, "m", 0, committed=False)
    s2 = m.alloc("k", 2, 32, "m", 0, committed=False)
    assert s1 == s2 and m.used_slots == 2


def test_abort_rolls_back_newest_reservation():
    m = make(8)
    A(m, "k1", 2)
    m.alloc("k2", 3, 48, "m", 0, committed=False)
    assert m.abort("k2") and m.head == 2 and m.used_slots == 2
    assert not m.abort("k1")  # committed chunks are not abortable


def test_explicit_evict_then_wrap_does_not_raise():
    m = make(8)
    A(m, "k1", 3), A(m, "k2", 3)
    assert m.evict_chunk("k1")
    # tail skipped the tombstone immediately
    assert m.tail == 3
    for i in range(10):
        A(m, f"n{i}", 3)


def test_eviction_listener_sees_every_path():
    m = make(6)
    seen = []
    m.add_eviction_listener(lambda meta: seen.append(meta.chunk_key))
    A(m, "k1", 3), A(m, "k2", 3), A(m, "k3", 3)
    m.evict_chunk("k2")
    assert seen == ["k1", "k2"]


def test_doc_registry_notified():
    docs = DocRegistry()
    m = make(6, docs)
    A(m, "k1", 3)
    m.store.get("k1").doc_ids.append("d")
    docs.insert(DocEntry("d", "t", chunk_keys=["k1"]))
    A(m, "k2", 3), A(m, "k3", 3)
    assert docs.get("d").status == "evicted" and docs.get("d").cached_mask == [False]


def test_save_load_roundtrip(tmp_path):
    m = make(8)
    A(m, "k1", 3), A(m, "k2", 2)
    m.alloc("pending", 1, 16, "m", 0, committed=False)
    p = str(tmp_path / "daser.index")
    m.save(p)
    m2 = make(8)
    m2.load(p)
    assert m2.store.get("k1") and m2.store.get("k2")
    # the half-written reservation is not resurrected
    assert m2.store.get("pending") is None
    assert m2.head == 5 and m2.tail == 0 and m2.used_slots == 5


def test_load_rejects_corrupt_ring(tmp_path):
    import msgpack

    m = make(8)
    A(m, "k1", 3)
    raw = msgpack.unpackb(m.to_bytes(), raw=False)
    raw["tail"] = 1  # points into the middle of a run
    p = tmp_path / "bad.index"
    p.write_bytes(msgpack.packb(raw, use_bin_type=True))
    m2 = make(8)
    with pytest.raises(RingInvariantError):
        m2.load(str(p))
    assert len(m2.store) == 0  # untouched on failure


def test_loads_a_reference_style_snapshot(tmp_path):
    """No "ext" map, occupancy inferred from the runs."""
    import msgpack

    m = make(8)
    A(m, "k1", 3), A(m, "k2", 2)
    raw = msgpack.unpackb(m.to_bytes(), raw=False)
    del raw["ext"]
    p = tmp_path / "ref.index"
    p.write_bytes(msgpack.packb(raw, use_bin_type=True))
    m2 = make(8)
    m2.load(str(p))
    assert m2.used_slots == 5


def test_random_ops_against_brute_force_model():
    rng = random.Random(7)
    for total in (5, 8, 13):
        m = make(total)
        live = {}  # key -> (start, n)
        for step in range(600):
            op = rng.random()
            if op < 0.7:
                n = rng.randint(1, total)
                key = f"c{total}_{step}"
                start = A(m, key, n)
                assert start + n <= total, "run straddles the end of the file"
                live = {k: v for k, v in live.items() if m.store.get(k) is not None}
                for k, (s, c) in live.items():
                    assert s + c <= start or start + n <= s, f"{key} overlaps {k}"
                live[key] = (start, n)
            elif op < 0.85 and live:
                key = rng.choice(sorted(live))
                m.evict_chunk(key)
                del live[key]
            elif m.used_slots:
                m.evict_oldest()
                live = {k: v for k, v in live.items() if m.store.get(k) is not None}
            assert 0 <= m.used_slots <= total
            assert sum(c for _, c in live.values()) <= m.used_slots
            assert set(live) == {c.chunk_key for c in m.store.iter_chunks()}
