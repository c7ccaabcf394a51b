"""Random operation sequences on the slot ring: invariants after every step, snapshot round trip.

The reference tests its ring with a handful of fixed scenarios (tests/server/test_chunk_manager.py);
two of its bugs (stale index entries after an eviction, a wrap over a live chunk when the ring is
full) only show under longer mixed sequences, which is what this test generates.
"""

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from daser_b200.server.chunk_manager import ChunkManager  # noqa: E402
from daser_b200.server.metadata_store import MetadataStore  # noqa: E402

TOTAL = 24

ops = st.lists(
    st.one_of(
        st.tuples(st.just("alloc"), st.integers(0, 40), st.integers(1, 9), st.booleans()),
        st.tuples(st.just("commit"), st.integers(0, 40)),
        st.tuples(st.just("evict"), st.integers(0, 40)),
        st.tuples(st.just("abort"), st.integers(0, 40)),
        st.tuples(st.just("snapshot")),
    ),
    min_size=1, max_size=120,
)


def _check(cm: ChunkManager, evicted: list[str], live_expected: set[str]) -> None:
    store = cm.store
    chunks = list(store.iter_chunks())
    # what the listeners reported and what the store holds add up to what was ever allocated
    assert {c.chunk_key for c in chunks} == live_expected
    # no two live chunks share a slot, none straddles the end of the file
    owner = {}
    for c in chunks:
        assert 0 <= c.start_slot and c.start_slot + c.num_slots <= TOTAL
        for s in range(c.start_slot, c.start_slot + c.num_slots):
            assert s not in owner, (c.chunk_key, owner.get(s))
            owner[s] = c.chunk_key
    assert 0 <= cm.used_slots <= TOTAL
    assert sum(c.num_slots for c in chunks) <= cm.used_slots  # padding and tombstones count as used
    if cm.used_slots == 0:
        assert not chunks
    # the occupied span runs from tail to head (mod TOTAL)
    if 0 < cm.used_slots < TOTAL:
        assert (cm.tail + cm.used_slots) % TOTAL == cm.head
    for c in chunks:
        assert cm.store.get_slot_entry(c.start_slot).chunk_key == c.chunk_key


@settings(max_examples=150, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(ops)
def test_ring_invariants_hold_under_mixed_operations(tmp_path_factory, sequence):
    cm = ChunkManager(TOTAL, MetadataStore(TOTAL))
    evicted: list[str] = []
    live: set[str] = set()
    cm.add_eviction_listener(lambda meta: (evicted.append(meta.chunk_key), live.discard(meta.chunk_key)))
    for op in sequence:
        kind = op[0]
        if kind == "alloc":
            _, k, n, committed = op
            key = f"k{k}"
            try:
                start = cm.alloc(key, n, n * 16, "m", 0, committed=committed)
            except ValueError:
                assert key in live  # the only refusal: the key exists (and is committed or differs)
            else:
                live.add(key)
                meta = cm.store.get(key)
                assert meta is not None and meta.start_slot == start
        elif kind == "commit":
            key = f"k{op[1]}"
            if cm.store.get(key) is not None:
                cm.store.mark_committed(key)
                assert cm.store.is_committed(key)
        elif kind == "evict":
            key = f"k{op[1]}"
            was_live = key in live
            assert cm.evict_chunk(key) == was_live
            assert cm.store.get(key) is None and key not in live
        elif kind == "abort":
            key = f"k{op[1]}"
            was_reservation = cm.store.get(key) is not None and not cm.store.is_committed(key)
            assert cm.abort(key) == was_reservation
            if was_reservation:
                assert cm.store.get(key) is None
        else:
            # a snapshot taken now and loaded into a fresh ring gives the committed chunks back at
            # the same slots, and the fresh ring keeps allocating without touching them
            path = str(tmp_path_factory.mktemp("snap") / "ring.index")
            cm.save(path)
            fresh = ChunkManager(TOTAL, MetadataStore(TOTAL))
            fresh.load(path)
            want = {c.chunk_key: (c.start_slot, c.num_slots) for c in cm.store.iter_chunks()
                    if cm.store.is_committed(c.chunk_key)}
            got = {c.chunk_key: (c.start_slot, c.num_slots) for c in fresh.store.iter_chunks()}
            assert got == want
            _check(fresh, [], set(got))
        _check(cm, evicted, live)
    # every key ever reported evicted is gone unless it was allocated again afterwards
    for key in set(evicted) - live:
        assert cm.store.get(key) is None
