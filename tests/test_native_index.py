"""The native token index against the pure-Python implementation (same digests, same answers)."""

import asyncio
import random
from array import array

import pytest
import xxhash

from daser_b200 import hashing
from daser_b200.retrieval.chunk_index import ChunkOffsetIndex
from daser_b200.server import native_index
from daser_b200.server.metadata_store import ChunkMeta

pytestmark = pytest.mark.skipif(not native_index.available(), reason="native index not built (python -m daser_b200.ops.build)")


def _meta(key, n, model="m", slot=0):
    return ChunkMeta(chunk_key=key, start_slot=slot, num_slots=-(-n // 16), token_count=n, pos_offset=0, model_id=model)


def test_digests_are_bit_identical_to_the_wheel():
    rng = random.Random(0)
    for n in (0, 1, 3, 4, 5, 16, 17, 31, 32, 33, 60, 61, 64, 100, 1000, 4097):
        toks = [rng.randrange(-(2**31), 2**31) for _ in range(n)]
        assert native_index.hash_tokens(toks) == xxhash.xxh3_128(array("i", toks).tobytes()).hexdigest()
    toks = [rng.randrange(128000) for _ in range(1000)]
    for block in (1, 7, 16, 64):
        want = [hashing.hash_tokens(toks[: (i + 1) * block]) for i in range(len(toks) // block)]
        assert native_index.prefix_digests(toks, block) == want
        want = [hashing.hash_tokens(toks[i * block : (i + 1) * block]) for i in range(len(toks) // block)]
        assert native_index.block_digests(toks, block) == want
    assert native_index.prefix_digests(toks[:5], 16) == []


def test_table_survives_growth_deletes_and_reinserts():
    rng = random.Random(1)
    table = native_index.DigestTable(4)
    ref = {}
    keys = [xxhash.xxh3_128(str(i).encode()).hexdigest() for i in range(3000)]
    for step in range(20000):
        k, tag = rng.choice(keys), rng.randrange(3)
        op = rng.random()
        if op < 0.55:
            table.put(tag, k, step)
            ref[(tag, k)] = step
        elif op < 0.85:
            assert table.delete(tag, k) == ((tag, k) in ref)
            ref.pop((tag, k), None)
        else:
            assert table.get(tag, k) == ref.get((tag, k), -1)
    assert len(table) == len(ref)
    for (tag, k), v in ref.items():
        assert table.get(tag, k) == v


def test_indexes_answer_like_the_python_path():
    rng = random.Random(2)
    nat, py = ChunkOffsetIndex(16, native=True), ChunkOffsetIndex(16, native=False)
    assert nat.native and not py.native
    prompt = [rng.randrange(50000) for _ in range(16 * 40)]
    loop = asyncio.new_event_loop()
    stored = []
    for idx, (nblk, model) in enumerate([(3, "m"), (10, "m"), (11, "other"), (25, "m"), (40, "other")]):
        key = hashing.hash_tokens(prompt[: nblk * 16])
        for ix in (nat, py):
            loop.run_until_complete(ix.insert(_meta(key, nblk * 16, model, slot=idx)))
        stored.append((key, nblk, model))
    loop.run_until_complete(nat.insert(_meta("not-a-digest", 16)))
    loop.run_until_complete(py.insert(_meta("not-a-digest", 16)))
    # a chunk in the middle of the prompt, registered with its anchor
    mid = prompt[16 * 12 : 16 * 20]
    mid_key = hashing.hash_tokens(mid)
    for ix in (nat, py):
        loop.run_until_complete(ix.insert(_meta(mid_key, len(mid))))
        ix.register_anchor(mid_key, hashing.hash_tokens(mid[:16]))

    def same(tokens, model):
        a, b = nat.lookup_sync(tokens, model), py.lookup_sync(tokens, model)
        assert [m.chunk_key for m in a] == [m.chunk_key for m in b]
        return a

    assert same(prompt, "m")[0].token_count == 25 * 16
    assert same(prompt, "other")[0].token_count == 40 * 16
    assert same(prompt[: 16 * 24 + 3], "m")[0].token_count == 10 * 16
    assert same(prompt[:40], "m") == []
    assert same(prompt, "nobody") == []
    for _ in range(50):
        cut = rng.randrange(0, len(prompt))
        same(prompt[:cut], rng.choice(["m", "other"]))
    hits_n, hits_p = nat.scan(prompt, "m"), py.scan(prompt, "m")
    assert [(h.meta.chunk_key, h.offset) for h in hits_n] == [(h.meta.chunk_key, h.offset) for h in hits_p]
    assert (mid_key, 16 * 12) in [(h.meta.chunk_key, h.offset) for h in hits_n]
    # removal and eviction paths keep both in step
    loop.run_until_complete(nat.remove(stored[3][0]))
    loop.run_until_complete(py.remove(stored[3][0]))
    nat.discard(stored[1][0])
    py.discard(stored[1][0])
    assert same(prompt, "m")[0].token_count == 3 * 16
    loop.close()


def test_scan_at_any_offset_matches_between_native_and_python():
    rng = random.Random(3)
    nat, py = ChunkOffsetIndex(16, native=True), ChunkOffsetIndex(16, native=False)
    prompt = [rng.randrange(50000) for _ in range(400)]
    loop = asyncio.new_event_loop()
    placed = [(21, 64), (100, 32), (133, 48)]  # offsets that are not multiples of 16
    for off, n in placed:
        toks = prompt[off : off + n]
        key = hashing.hash_tokens(toks)
        for ix in (nat, py):
            loop.run_until_complete(ix.insert(_meta(key, n)))
            ix.register_anchor(key, hashing.hash_tokens(toks[:16]))
    loop.close()
    for ix in (nat, py):
        assert ix.scan(prompt, "m") == []  # none of them sits on a block boundary
        got = [(h.offset, h.meta.token_count) for h in ix.scan(prompt, "m", any_offset=True)]
        assert got == placed
    assert native_index.window_digests(prompt[:40], 16) == [hashing.hash_tokens(prompt[i : i + 16]) for i in range(25)]
    assert native_index.window_digests(prompt[:10], 16) == []
