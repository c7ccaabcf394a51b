"""HBM tier bookkeeping (runs on CPU memory: the arena is just a tensor)."""

import pytest
import torch

from daser_b200.kv.hbm_store import HBMStore


def test_lru_and_contiguity():
    s = HBMStore(slot_size=64, capacity_slots=8, device=torch.device("cpu"))
    src = torch.arange(64 * 8, dtype=torch.int64).to(torch.uint8)
    assert s.admit("a", src, 0, 64 * 3) and s.admit("b", src, 64, 64 * 3)
    s.end_step()
    assert s.lookup("zz") is None
    pa = s.lookup("a")  # 'a' is now most recently used
    assert pa == s.arena.data_ptr()
    assert s.admit("c", src, 0, 64 * 4)  # needs eviction: 'b' is LRU, but freeing b gives 3+2=5 contiguous
    assert "b" not in s and "a" in s and "c" in s
    assert s.used_slots == 7
    # contents survive
    first = (s.lookup("c") - s.arena.data_ptr()) // 64
    assert torch.equal(s.arena[first * 64 : first * 64 + 256], src[:256])
    assert not s.admit("huge", src, 0, 64 * 9)
    s.end_step()
    assert s.evict("a") and not s.evict("a")
    assert s.admit("d", src, 0, 64 * 4)  # free runs are [0,3) and [7,8): 'c' has to go too
    assert len(s) == 1 and s.stats()["used_slots"] == 4


def test_fragmentation_evicts_until_a_run_fits():
    s = HBMStore(32, 6, torch.device("cpu"))
    src = torch.zeros(32 * 6, dtype=torch.uint8)
    for k in "abc":
        s.admit(k, src, 0, 64)
    s.end_step()
    s.evict("b")  # hole of 2 in the middle
    assert s.admit("d", src, 0, 32 * 4)  # must evict 'a' (LRU) to merge [0,4)
    assert "a" not in s and "c" in s


def test_entries_used_by_the_current_step_are_not_evicted():
    s = HBMStore(16, 4, torch.device("cpu"))
    src = torch.zeros(64, dtype=torch.uint8)
    s.admit("a", src, 0, 32)
    s.admit("b", src, 0, 32)
    s.end_step()
    assert s.lookup("a") is not None  # this step reads 'a'
    off = s.reserve("c", 32)          # 'b' can go
    assert off is not None and "b" not in s and "a" in s
    assert s.reserve("d", 32) is None  # would need 'a' or 'c', both in use by this step
    s.end_step()
    assert s.reserve("d", 32) is not None


def test_clear_forgets_everything_and_frees_the_arena():
    import torch

    from daser_b200.kv.hbm_store import HBMStore

    tier = HBMStore(64, 8, torch.device("cpu"))
    src = torch.arange(64 * 8, dtype=torch.uint8)
    for i in range(4):
        assert tier.admit(f"k{i}", src, 0, 128)
    assert tier.used_slots == 8 and len(tier) == 4
    assert tier.clear() == 4
    assert len(tier) == 0 and tier.used_slots == 0 and tier.lookup("k0") is None
    assert tier.reserve("big", 64 * 8) == 0  # the whole arena is one free run again


def test_tier_invariants_under_random_operations():
    """Random reserve / admit / lookup / evict / end_step sequences: entries never overlap, free
    runs and entries tile the arena exactly, and nothing looked up in the current step is evicted."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings
    from hypothesis import strategies as st

    import torch

    from daser_b200.kv.hbm_store import HBMStore

    CAP, SLOT = 16, 32
    op = st.one_of(
        st.tuples(st.just("reserve"), st.integers(0, 11), st.integers(1, 6)),
        st.tuples(st.just("admit"), st.integers(0, 11), st.integers(1, 6)),
        st.tuples(st.just("lookup"), st.integers(0, 11)),
        st.tuples(st.just("evict"), st.integers(0, 11)),
        st.tuples(st.just("end_step")),
        st.tuples(st.just("clear")),
    )

    @settings(max_examples=200, deadline=None, derandomize=True)
    @given(st.lists(op, min_size=1, max_size=80))
    def run(sequence):
        tier = HBMStore(SLOT, CAP, torch.device("cpu"))
        src = torch.arange(SLOT * CAP, dtype=torch.int64).to(torch.uint8)
        pinned_this_step: set[str] = set()
        sizes: dict[str, int] = {}
        for o in sequence:
            kind = o[0]
            if kind in ("reserve", "admit"):
                key, n = f"k{o[1]}", o[2]
                n = sizes.get(key, n) if key in tier else n
                if kind == "reserve":
                    off = tier.reserve(key, n * SLOT)
                    ok = off is not None
                else:
                    ok = tier.admit(key, src, 0, n * SLOT)
                if ok:
                    sizes[key] = n
                    pinned_this_step.add(key)
                    assert key in tier
            elif kind == "lookup":
                key = f"k{o[1]}"
                ptr = tier.lookup(key)
                assert (ptr is not None) == (key in tier)
                if ptr is not None:
                    pinned_this_step.add(key)
                    assert (ptr - tier.arena.data_ptr()) % SLOT == 0
            elif kind == "evict":
                key = f"k{o[1]}"
                had = key in tier
                assert tier.evict(key) == had
                pinned_this_step.discard(key)
            elif kind == "end_step":
                tier.end_step()
                pinned_this_step.clear()
            else:
                tier.clear()
                pinned_this_step.clear()
            # whatever was touched in this step is still there
            for key in pinned_this_step:
                assert key in tier, (key, sequence)
            # entries and free runs tile the arena exactly once
            spans = sorted([(f, n) for f, n in tier._chunks.values()] + list(tier._free))
            pos = 0
            for first, n in spans:
                assert first == pos and n > 0
                pos += n
            assert pos == CAP
            assert tier.used_slots == sum(n for _, n in tier._chunks.values()) <= CAP

    run()


def test_trimmed_prefix_hit_does_not_shadow_the_whole_chunk(tmp_path):
    """A prompt equal to a stored chunk loads one slot fewer than the chunk has (the engine must
    compute at least one token).  That short load must not be cached under the chunk's key: a
    later, longer prompt reads the whole chunk and must get every block right."""
    from conftest import LiveControlPlane
    from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
    from daser_b200.kv.hbm_store import HBMStore
    from daser_b200.kv.layout import KVGeometry

    L, H, D, B = 2, 2, 32, 16
    geo = KVGeometry(num_layers=L, num_kv_heads=H, head_dim=D, block_tokens=B, dtype_bytes=2, codec="raw")
    lp = LiveControlPlane(tmp_path, total_slots=64, slot_size=geo.slot_size).start()
    torch.manual_seed(3)
    pool = torch.randn(L, 24, 2, H, B, D).to(torch.bfloat16)
    host = HBMStore(geo.slot_size, 16, torch.device("cpu"))
    worker = WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool, [1.0] * (D // 2)),
                        io_backend="posix", staging_slots=8, host_store=host)
    sched = SchedulerHalf(lp.socket_path, B, "m")

    def step(req, fn):
        fn()
        meta = sched.build_connector_meta([req])
        worker.bind_connector_metadata(meta)
        worker.start_load_kv()
        worker.wait_for_save()
        worker.clear_connector_metadata()
        sched.request_finished(req)
        return meta

    try:
        tokens = list(range(500, 500 + 4 * B))
        # another chunk right behind it in the arena and in the file, so an over-read is visible
        other = list(range(900, 900 + 4 * B))
        for rid, toks, blocks in (("s1", tokens, [1, 2, 3, 4]), ("s2", other, [5, 6, 7, 8])):
            def cold(rid=rid, toks=toks, blocks=blocks):
                assert sched.get_num_new_matched_tokens(rid, toks + [1], 0) == (0, False)
                sched.update_state_after_alloc(rid, blocks, 0)
            step(rid, cold)
        host.clear()  # cold tier: the next loads come from the file
        want = pool[:, [1, 2, 3, 4]].clone()

        def trimmed():
            n, _ = sched.get_num_new_matched_tokens("t1", tokens, 0)  # the prompt IS the chunk
            assert n == 3 * B
            sched.update_state_after_alloc("t1", [10, 11, 12], n)
        meta = step("t1", trimmed)
        assert len(meta.reqs_to_load[0].block_ids) == 3
        assert torch.equal(pool[:, [10, 11, 12]], want[:, :3])

        def full():
            n, _ = sched.get_num_new_matched_tokens("t2", tokens + [7, 8, 9], 0)
            assert n == 4 * B
            sched.update_state_after_alloc("t2", [14, 15, 16, 17, 18], n)
        step("t2", full)
        assert torch.equal(pool[:, [14, 15, 16, 17]], want)
        # and the whole chunk is what the tier now holds
        assert host.lookup(meta.reqs_to_load[0].chunk_key, 4) is not None
        host.end_step()
    finally:
        worker.shutdown()
        sched.close()
        lp.stop()


def test_a_chunk_longer_than_the_staging_arena_is_stored_and_restored_in_pieces(tmp_path):
    """Ten blocks through an arena of four slots: three rounds on the way out, three waves on the
    way back, every block exact; a second, short chunk shares the step."""
    from conftest import LiveControlPlane
    from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
    from daser_b200.kv.layout import KVGeometry

    L, H, D, B = 2, 2, 32, 16
    geo = KVGeometry(num_layers=L, num_kv_heads=H, head_dim=D, block_tokens=B, dtype_bytes=2, codec="raw")
    lp = LiveControlPlane(tmp_path, total_slots=64, slot_size=geo.slot_size).start()
    torch.manual_seed(5)
    pool = torch.randn(L, 40, 2, H, B, D).to(torch.bfloat16)
    worker = WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool, [1.0] * (D // 2)),
                        io_backend="posix", staging_slots=4)
    sched = SchedulerHalf(lp.socket_path, B, "m")

    def step(reqs, fn):
        fn()
        meta = sched.build_connector_meta(reqs)
        worker.bind_connector_metadata(meta)
        worker.start_load_kv()
        worker.wait_for_save()
        worker.clear_connector_metadata()
        for r in reqs:
            sched.request_finished(r)
        return meta

    try:
        long_toks = list(range(100, 100 + 10 * B))
        short_toks = list(range(700, 700 + 2 * B))
        src_long, src_short = list(range(1, 11)), [11, 12]

        def cold():
            assert sched.get_num_new_matched_tokens("a", long_toks + [1], 0) == (0, False)
            sched.update_state_after_alloc("a", src_long + [13], 0)
            assert sched.get_num_new_matched_tokens("b", short_toks + [1], 0) == (0, False)
            sched.update_state_after_alloc("b", src_short + [14], 0)
        step(["a", "b"], cold)
        want_long, want_short = pool[:, src_long].clone(), pool[:, src_short].clone()
        dst_long, dst_short = list(range(20, 30)), [30, 31]

        def warm():
            n, _ = sched.get_num_new_matched_tokens("c", long_toks + [1, 2], 0)
            assert n == 10 * B
            sched.update_state_after_alloc("c", dst_long + [32], n)
            n, _ = sched.get_num_new_matched_tokens("d", short_toks + [1, 2], 0)
            assert n == 2 * B
            sched.update_state_after_alloc("d", dst_short + [33], n)
        step(["c", "d"], warm)
        assert torch.equal(pool[:, dst_long], want_long)
        assert torch.equal(pool[:, dst_short], want_short)
        assert not worker.take_load_errors()
    finally:
        worker.shutdown()
        sched.close()
        lp.stop()


def test_write_behind_stores_commit_later_and_survive_a_failed_write(tmp_path):
    """``write_behind``: ``wait_for_save`` returns with the file write in flight; the chunk is
    committed when its half of the arena is needed again, before a load that uses the arena, or at
    ``flush_stores``.  A write that fails aborts that chunk only."""
    from conftest import LiveControlPlane
    from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
    from daser_b200.kv.layout import KVGeometry

    L, H, D, B = 2, 2, 32, 16
    geo = KVGeometry(num_layers=L, num_kv_heads=H, head_dim=D, block_tokens=B, dtype_bytes=2, codec="raw")
    lp = LiveControlPlane(tmp_path, total_slots=64, slot_size=geo.slot_size).start()
    torch.manual_seed(7)
    pool = torch.randn(L, 40, 2, H, B, D).to(torch.bfloat16)
    worker = WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool, [1.0] * (D // 2)),
                        io_backend="posix", staging_slots=8, write_behind=True)
    sched = SchedulerHalf(lp.socket_path, B, "m")

    def store(rid, toks, blocks):
        assert sched.get_num_new_matched_tokens(rid, toks + [1], 0) == (0, False)
        sched.update_state_after_alloc(rid, blocks + [39], 0)
        meta = sched.build_connector_meta([rid])
        worker.bind_connector_metadata(meta)
        worker.wait_for_save()
        worker.clear_connector_metadata()
        sched.request_finished(rid)
        return meta.reqs_to_store[0].chunk_key

    def visible(toks):
        n, _ = sched.get_num_new_matched_tokens("probe", toks + [1, 2], 0)
        sched.request_finished("probe")
        return n == len(toks)

    try:
        chunks = [list(range(100 * (i + 1), 100 * (i + 1) + 3 * B)) for i in range(4)]
        blocks = [[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11, 12]]
        ka = store("a", chunks[0], blocks[0])
        assert worker.pending_store_keys() == {ka} and not visible(chunks[0])
        kb = store("b", chunks[1], blocks[1])            # the other half of the arena: a is still in flight
        assert worker.pending_store_keys() == {ka, kb}
        worker.flush_stores()
        assert not worker.pending_store_keys() and visible(chunks[0]) and visible(chunks[1])
        worker._xfer.engine.inject_fault(1, err_no=5)     # the next write fails
        kc = store("c", chunks[2], blocks[2])
        kd = store("d", chunks[3], blocks[3])
        assert worker.pending_store_keys() == {kc, kd}
        worker.flush_stores()
        assert not visible(chunks[2]) and visible(chunks[3])  # c's write failed: aborted, never visible
        store("c2", chunks[2], blocks[2])                # and can be stored again; stays pending for now
        # a load that uses the arena completes what is pending first
        want = pool[:, blocks[0]].clone()
        n, _ = sched.get_num_new_matched_tokens("r", chunks[0] + [1, 2], 0)
        assert n == 3 * B
        sched.update_state_after_alloc("r", [20, 21, 22, 23], n)
        worker.bind_connector_metadata(sched.build_connector_meta(["r"]))
        worker.start_load_kv()
        worker.clear_connector_metadata()
        sched.request_finished("r")
        assert not worker.pending_store_keys() and visible(chunks[2])
        assert torch.equal(pool[:, [20, 21, 22]], want)
    finally:
        worker.shutdown()
        sched.close()
        lp.stop()


@pytest.mark.parametrize("staging_slots,write_behind", [(2, False), (3, True), (5, False), (8, True)])
def test_random_chunks_through_small_arenas_come_back_exact(tmp_path, staging_slots, write_behind):
    """Chunks of 1..12 blocks, several per step, through arenas smaller than most of them, with and
    without write-behind: every chunk is restored bit for bit into other blocks."""
    import random

    from conftest import LiveControlPlane
    from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
    from daser_b200.kv.layout import KVGeometry

    L, H, D, B = 2, 1, 32, 16
    geo = KVGeometry(num_layers=L, num_kv_heads=H, head_dim=D, block_tokens=B, dtype_bytes=2, codec="raw")
    lp = LiveControlPlane(tmp_path, total_slots=256, slot_size=geo.slot_size).start()
    rng = random.Random(staging_slots * 7 + write_behind)
    torch.manual_seed(staging_slots)
    n_blocks = 160
    pool = torch.randn(L, n_blocks, 2, H, B, D).to(torch.bfloat16)
    worker = WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool, [1.0] * (D // 2)),
                        io_backend="posix", staging_slots=staging_slots, write_behind=write_behind)
    sched = SchedulerHalf(lp.socket_path, B, "m")

    def step(reqs):
        meta = sched.build_connector_meta(reqs)
        worker.bind_connector_metadata(meta)
        worker.start_load_kv()
        worker.wait_for_save()
        worker.clear_connector_metadata()
        for r in reqs:
            sched.request_finished(r)

    try:
        free = list(range(1, n_blocks))
        chunks = []
        for i in range(9):
            nb = rng.randint(1, 12)
            toks = [rng.randrange(1, 30000) for _ in range(nb * B)]
            blocks = [free.pop() for _ in range(nb)]
            chunks.append((f"s{i}", toks, blocks, pool[:, blocks].clone()))
        for group in (chunks[:4], chunks[4:7], chunks[7:]):
            for rid, toks, blocks, _ in group:
                assert sched.get_num_new_matched_tokens(rid, toks + [1], 0) == (0, False)
                sched.update_state_after_alloc(rid, blocks + [0], 0)
            step([rid for rid, *_ in group])
        worker.flush_stores()
        loads = []
        for i, (rid, toks, _, want) in enumerate(chunks):
            nb = len(toks) // B
            dst = [free.pop() for _ in range(nb)]
            n, _ = sched.get_num_new_matched_tokens(f"l{i}", toks + [1, 2], 0)
            assert n == nb * B
            sched.update_state_after_alloc(f"l{i}", dst + [0], n)
            loads.append((f"l{i}", dst, want))
        step([rid for rid, *_ in loads[:5]])
        step([rid for rid, *_ in loads[5:]])
        for rid, dst, want in loads:
            assert torch.equal(pool[:, dst], want), rid
        assert not worker.take_load_errors()
    finally:
        worker.shutdown()
        sched.close()
        lp.stop()
