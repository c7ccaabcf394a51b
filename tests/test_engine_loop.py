"""The engine loop: concurrent callers share the engine's steps (continuous batching)."""

import random
import threading
import time

import pytest

from conftest import LiveControlPlane
from daser_b200.engine.loop import EngineLoop
from daser_b200.engine.rag_cpu import CpuRagEngine
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import PRESETS
from daser_b200.position import RopeReencoder


@pytest.fixture
def engine(tmp_path):
    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=256, slot_size=geo.slot_size, num_layers=cfg.num_layers,
                          num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, dtype_bytes=4)
    lp.plane.position = RopeReencoder(cfg.head_dim, cfg.rope_theta)
    lp.start()
    eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=256)
    yield eng
    eng.close()
    lp.stop()


def test_concurrent_requests_share_steps_and_match_sequential_results(engine):
    cfg = engine.cfg
    rng = random.Random(0)
    chunks = [[rng.randrange(cfg.vocab_size) for _ in range(32)] for _ in range(4)]
    for c in chunks:
        engine.store_chunk(c)
    reqs = [([rng.choice(chunks), rng.choice(chunks)], [rng.randrange(cfg.vocab_size) for _ in range(6)])
            for _ in range(6)]
    want = [engine.generate(c, q, max_new_tokens=5).generated for c, q in reqs]
    free_before = engine.blocks.num_free

    loop = EngineLoop(engine)
    try:
        streams = [[] for _ in reqs]
        futs = [loop.submit(c, q, 5, on_token=streams[i].append) for i, (c, q) in enumerate(reqs)]
        # an engine call from another thread is slotted in between two steps
        key = loop.call("store_chunk", [rng.randrange(cfg.vocab_size) for _ in range(16)]).result(60)
        done = [f.result(60) for f in futs]
    finally:
        loop.close()
    assert [r.generated for r in done] == want            # batching changes the schedule, not the tokens
    assert streams == want                                 # every token was reported, in order
    assert all(r.restored_chunks == 2 for r in done)
    assert loop.max_batch > 1                              # requests really overlapped
    assert loop.steps < sum(len(w) for w in want)          # fewer steps than one request at a time needs
    assert isinstance(key, str) and engine.blocks.num_free == free_before


def test_requests_arriving_while_others_decode_join_the_batch(engine):
    cfg = engine.cfg
    loop = EngineLoop(engine)
    try:
        first = loop.submit([], [1, 2, 3], 40)
        started = threading.Event()
        got = []
        second = None

        def late():
            nonlocal second
            time.sleep(0.05)
            second = loop.submit([], [4, 5, 6], 3, on_token=lambda t: (got.append(t), started.set()))

        t = threading.Thread(target=late)
        t.start()
        t.join()
        r2 = second.result(60)
        assert not first.done() or len(first.result().generated) == 40   # the short one did not wait for the long one
        r1 = first.result(60)
    finally:
        loop.close()
    assert len(r1.generated) == 40 and len(r2.generated) == 3 and got == r2.generated
    assert r2.generated == engine.generate([], [4, 5, 6], max_new_tokens=3).generated
    assert cfg.block_tokens == 16


def test_a_failing_step_fails_everything_in_flight_and_later_calls():
    class Broken:
        def __init__(self):
            self.q = []

        def submit(self, req):
            self.q.append(req)

        def has_work(self):
            return bool(self.q)

        def step(self):
            raise RuntimeError("device status word set")

    loop = EngineLoop(Broken())
    fut = loop.submit([], [1], 2)
    with pytest.raises(RuntimeError, match="status word"):
        fut.result(10)
    assert loop.failed is not None
    with pytest.raises(RuntimeError, match="not running"):
        loop.submit([], [1], 1).result(1)
    with pytest.raises(RuntimeError, match="not running"):
        loop.call("store_chunk", [1]).result(1)
    loop.close()
    with pytest.raises(TypeError):
        EngineLoop(object())


def test_a_callers_error_in_call_does_not_stop_the_loop(engine):
    loop = EngineLoop(engine)
    try:
        for bad in (([[1, 2, 3]], [4], 1), ([], [], 1), ([], [4], 0)):      # ragged segment, no query, nothing to generate
            with pytest.raises(ValueError):
                loop.submit(*bad).result(5)
        with pytest.raises(ValueError):
            loop.call("store_chunk", [1, 2, 3]).result(30)   # not a whole number of blocks
        assert len(loop.submit([], [9, 9], 2).result(60).generated) == 2
    finally:
        loop.close()


def test_a_request_that_cannot_fit_is_given_up_alone_and_one_that_must_wait_waits(tmp_path):
    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=64, slot_size=geo.slot_size, num_layers=cfg.num_layers,
                          num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, dtype_bytes=4)
    lp.start()
    eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=8)     # 128 tokens of KV in all
    loop = EngineLoop(eng)
    try:
        a = loop.submit([], list(range(1, 60)), 30)          # 89 tokens: 6 blocks
        b = loop.submit([], list(range(1, 50)), 20)          # 69 tokens: 5 blocks, does not fit beside a
        huge = loop.submit([], list(range(1, 120)), 40)      # 159 tokens: 10 blocks, never fits
        ra = a.result(120)
        rb = b.result(120)                                   # waited for a's blocks, then ran
        with pytest.raises(MemoryError, match="KV blocks"):
            huge.result(120)
        assert len(ra.generated) == 30 and len(rb.generated) == 20
        assert loop.failed is None and eng.blocks.num_free == 8
        assert len(loop.submit([], [5, 6, 7], 2).result(60).generated) == 2      # the loop lives on
    finally:
        loop.close()
    with pytest.raises(MemoryError):
        eng.generate([], list(range(1, 120)), max_new_tokens=40)
    assert eng.blocks.num_free == 8
    eng.close()
    lp.stop()


def test_cancelled_requests_leave_the_engine_and_return_their_blocks(engine):
    import asyncio

    from daser_b200.service.vllm_client import NativeEngineClient

    loop = EngineLoop(engine)
    free = engine.blocks.num_free
    try:
        got = []
        long_one = loop.submit([], [1, 2, 3], 400, on_token=got.append)
        other = loop.submit([], [4, 5, 6], 5)
        while len(got) < 3:
            time.sleep(0.01)
        loop.cancel(long_one)
        with pytest.raises(RuntimeError, match="cancelled"):
            long_one.result(30)
        assert len(other.result(60).generated) == 5            # the neighbour was not disturbed
        assert len(got) < 400
        loop.cancel(other)                                     # finished already: nothing happens
        assert loop.call("has_work").result(10) is False and engine.blocks.num_free == free
        assert engine.abort("no-such-request") is False
    finally:
        loop.close()

    # the same through the streaming client: a consumer that stops reading cancels the request
    client = NativeEngineClient(engine, lambda ids: "".join(chr(65 + i % 26) for i in ids), batching=True)

    async def read_three():
        agen = client.completion_stream([1, 2, 3], {"max_tokens": 400})
        seen = []
        async for item in agen:
            seen.append(item)
            if len(seen) == 3:
                break
        await agen.aclose()
        for _ in range(200):                                   # the abort happens between two steps
            if not engine.has_work():
                break
            await asyncio.sleep(0.01)
        await client.close()
        return seen

    seen = asyncio.run(read_three())
    assert len(seen) == 3 and not engine.has_work() and engine.blocks.num_free == free


def test_per_sequence_block_limit_rejects_alone(engine):
    """The CUDA engine's runner has block tables of a fixed width; the shared admission code turns a
    request beyond it away (here with the limit set on the oracle engine)."""
    engine.max_blocks_per_seq = 4
    try:
        with pytest.raises(MemoryError, match="per sequence"):
            engine.generate([], list(range(1, 70)), max_new_tokens=10)     # 79 tokens: 5 blocks
        assert len(engine.generate([], list(range(1, 40)), max_new_tokens=10).generated) == 10
    finally:
        engine.max_blocks_per_seq = None


def test_composed_chunks_also_work_through_the_engine_loop(engine):
    from daser_b200 import metrics

    engine.compose_after = 2
    rng = random.Random(3)
    a, b = ([rng.randrange(engine.cfg.vocab_size) for _ in range(32)] for _ in range(2))
    loop = EngineLoop(engine)
    try:
        first = loop.submit([a, b], [1, 2, 3], 3).result(60)
        loop.submit([a, b], [1, 2, 3], 3).result(60)              # second sighting: [a, b] gets stored
        hits0 = metrics.snapshot().get("connector.composed_hits", 0)
        third = loop.submit([a, b], [1, 2, 3], 3).result(60)
    finally:
        loop.close()
        engine.compose_after = 0
    assert metrics.snapshot().get("connector.composed_hits", 0) == hits0 + 1
    assert third.restored_chunks == 1 and third.generated == first.generated and third.asked == [a, b]


def test_back_pressure_refuses_at_once_above_the_limit(engine):
    from daser_b200.engine.loop import QueueFull

    loop = EngineLoop(engine, max_in_flight=2)
    try:
        a = loop.submit([], [1, 2, 3], 60)
        b = loop.submit([], [4, 5, 6], 60)
        c = loop.submit([], [7, 8, 9], 2)
        with pytest.raises(QueueFull, match="limit 2"):
            c.result(1)
        a.result(60), b.result(60)
        assert len(loop.submit([], [7, 8, 9], 2).result(60).generated) == 2      # room again
    finally:
        loop.close()


def test_a_future_cancelled_by_its_owner_does_not_stop_the_loop(engine):
    """An asyncio wrapper that is cancelled cancels the future underneath it at once; when the
    request then finishes (or is aborted) the loop must shrug, not die on the dead future."""
    loop = EngineLoop(engine)
    try:
        doomed = loop.submit([], [1, 2, 3], 4)
        assert doomed.cancel()                                # still pending: the owner wins
        other = loop.submit([], [4, 5, 6], 3)
        assert len(other.result(60).generated) == 3
        time.sleep(0.2)                                       # the doomed request runs out meanwhile
        assert loop.failed is None
        assert len(loop.submit([], [7, 8], 2).result(60).generated) == 2
        late = loop.call("has_work")
        late.cancel()
        assert loop.call("has_work").result(10) in (True, False) and loop.failed is None
    finally:
        loop.close()
    assert engine.blocks.num_free == 256


def test_close_aborts_what_outlives_its_patience(engine):
    loop = EngineLoop(engine)
    long_one = loop.submit([], [1, 2, 3], 3000)
    time.sleep(0.1)
    t0 = time.time()
    loop.close(timeout_s=0.3)
    assert time.time() - t0 < 5 and not loop._thread.is_alive()
    with pytest.raises(RuntimeError, match="closed"):
        long_one.result(1)
    assert not engine.has_work() and engine.blocks.num_free == 256
