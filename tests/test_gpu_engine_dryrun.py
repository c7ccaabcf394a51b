"""The CUDA engine's host-side control flow, run without a GPU.

``GpuRagEngine`` is Python around a model runner and a KV backend.  Here the runner is replaced by a
recorder that "samples" a deterministic function of what it was asked to compute, the KV backend by
the PyTorch one on a host pool, and the CUDA events by stubs; scheduler half, worker half, block
allocator, store file and control plane are the real ones.  What is checked is which work the
engine asks for: what is restored and what is computed, where, with which sampling fields, and what
happens to queues and blocks.  (Numerics of the real runner: ``tests/test_gpu_engine.py``.)"""

import random

import pytest
import torch

from conftest import LiveControlPlane
from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
from daser_b200.engine.loop import EngineLoop
from daser_b200.engine.rag_cpu import BlockAllocator
from daser_b200.engine.rag_gpu import GpuRagEngine
from daser_b200.engine.request import RagRequest
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import PRESETS, TorchPagedKV


class _Event:
    def record(self):
        pass

    def elapsed_time(self, other):
        return 0.0


class _Runner:
    """Records every forward; the "sampled" token of a sequence is a hash of its last token and position."""

    max_tokens, max_seqs, max_blocks = 64, 4, 32
    layer_groups = [(0, 2)]
    layers = range(2)
    h2d_bytes = 0
    status = None

    def __init__(self):
        self.calls = []

    def stage_inputs(self, seqs):
        return [dict(s, tokens=list(s["tokens"]), block_table=list(s["block_table"])) for s in seqs]

    def forward(self, seqs, gate=None):
        if gate is not None:
            for g in range(len(self.layer_groups)):
                gate(g)  # the restore pieces, in order, in front of the layers that read them
        self.calls.append(seqs)
        return torch.tensor([(s["tokens"][-1] * 31 + s["start_pos"] + len(s["tokens"])) % 1000 for s in seqs])

    def check_status(self):
        pass


@pytest.fixture
def engine(tmp_path):
    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    eng = GpuRagEngine.__new__(GpuRagEngine)                 # not __init__: that needs a GPU
    eng.cfg, eng.geo, eng.tp, eng.rank, eng.tp_ctx, eng.pp_link = cfg, geo, 1, 0, None, None
    eng.compose_after = eng.repair_tokens = 0
    eng.interleave_decode = True
    eng.runner = _Runner()
    eng.blocks = BlockAllocator(32)
    eng.max_blocks_per_seq = eng.runner.max_blocks
    pool = TorchPagedKV(cfg, 32)
    eng.sched = SchedulerHalf(lp.socket_path, cfg.block_tokens, "default")
    eng.worker = WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool.data, cfg.inv_freq()),
                            io_backend="posix")
    eng.hbm = eng.host = None
    eng.kv_backend = eng.worker.kv
    eng.kv_backend.h2d_bytes = 0
    eng.waiting, eng.running, eng._n = [], [], 0
    eng._ev = [_Event() for _ in range(4)]
    eng._restore_stream, eng._group_ev, eng._kv_epoch, eng.h2d_bytes = None, [], 0, 0
    yield eng
    eng.worker.shutdown()
    eng.sched.close()
    lp.stop()


def _computed(calls):
    """(start_pos, number of tokens) of every sequence of every forward, in order."""
    return [(s["start_pos"], len(s["tokens"])) for seqs in calls for s in seqs]


def test_restore_compute_repair_and_sampling_fields(engine):
    rng = random.Random(0)
    a, b = ([rng.randrange(1000) for _ in range(32)] for _ in range(2))
    engine.store_chunk(a)
    assert _computed(engine.runner.calls) == [(0, 32)] and engine.blocks.num_free == 32
    engine.runner.calls.clear()
    seen = []
    req = engine.generate([a, b], [5, 6, 7], max_new_tokens=3, temperature=0.7, seed=9, on_token=seen.append)
    # chunk a restored (no forward); chunk b and the query behind it go through the model as one run
    # of 35 tokens at b's offset (one pass over the weights, not two), then two decode steps
    assert req.restored_chunks == 1 and _computed(engine.runner.calls) == [(32, 35), (67, 1), (68, 1)]
    assert seen == req.generated and len(seen) == 3 and req.finish_reason == "length"
    sampled = [s for seqs in engine.runner.calls for s in seqs]
    assert all(s["temperature"] == 0.7 for s in sampled)
    assert len({s["seed"] for s in sampled}) == 3            # a fresh seed per step, derived from the request's
    # a missed chunk in FRONT of a restored one is a run of its own, and samples nothing
    engine.runner.calls.clear()
    c = [rng.randrange(1000) for _ in range(32)]
    req = engine.generate([c, a], [5, 6, 7], max_new_tokens=1, temperature=0.7, seed=9)
    assert req.restored_chunks == 1 and _computed(engine.runner.calls) == [(0, 32), (64, 3)]
    assert "temperature" not in engine.runner.calls[0][0] and engine.runner.calls[1][0]["temperature"] == 0.7
    engine.runner.calls.clear()
    engine.generate([], [5, 6], max_new_tokens=2, temperature=0.7, seed=1, top_k=40, top_p=0.9)
    assert all(s["top_k"] == 40 and s["top_p"] == 0.9 for seqs in engine.runner.calls for s in seqs)
    assert engine.blocks.num_free == 32 and not engine.has_work()
    # head repair: the restored chunk behind other context gets its first tokens recomputed in place
    engine.store_chunk(b)
    engine.runner.calls.clear()
    engine.repair_tokens = 8
    req = engine.generate([b, a], [1], max_new_tokens=1)
    assert req.restored_chunks == 2 and _computed(engine.runner.calls) == [(32, 8), (64, 1)]
    engine.repair_tokens = 0
    # stop tokens end the request early and free its blocks
    first = engine.generate([], [9, 9], max_new_tokens=4).generated
    cut = engine.generate([], [9, 9], max_new_tokens=4, stop_token_ids=[first[1]])
    assert cut.generated == first[:2] and cut.finish_reason == "stop" and engine.blocks.num_free == 32


def test_composed_chunks_admission_abort_and_the_engine_loop(engine):
    rng = random.Random(1)
    a, b = ([rng.randrange(1000) for _ in range(16)] for _ in range(2))
    engine.compose_after = 2
    engine.generate([a, b], [3], max_new_tokens=1)
    engine.generate([a, b], [3], max_new_tokens=1)            # second sighting: [a, b] stored as one chunk
    engine.runner.calls.clear()
    req = engine.generate([a, b], [3], max_new_tokens=1)
    assert req.restored_chunks == 1 and _computed(engine.runner.calls) == [(32, 1)]
    engine.compose_after = 0
    # admission: 32 blocks of 16 tokens in the pool, 32 per sequence at most
    with pytest.raises(MemoryError, match="per sequence"):
        engine.generate([], [1] * 600, max_new_tokens=1)
    engine.max_blocks_per_seq = 64
    with pytest.raises(MemoryError, match="pool has 32 free"):
        engine.generate([], [1] * 600, max_new_tokens=1)
    assert engine.blocks.num_free == 32
    # two requests that do not fit side by side: the second waits, is aborted while waiting
    r1 = engine.submit(RagRequest([], [1] * 300, 4))
    r2 = engine.submit(RagRequest([], [2] * 300, 4))
    engine.step()
    assert r1 in engine.running and r2 in engine.waiting
    engine.step()                                              # r2 still lacks blocks: r1 decodes instead
    assert len(r1.generated) == 2 and not r2.generated
    assert engine.abort(r2.req_id) and r2.error == "aborted" and r2.done
    while not r1.done:
        engine.step()
    assert engine.blocks.num_free == 32 and not engine.has_work()
    # and under the engine loop: decode steps carry every running request together
    engine.runner.calls.clear()
    loop = EngineLoop(engine)
    try:
        futs = [loop.submit([], [i + 1] * 10, 6) for i in range(3)]
        done = [f.result(30) for f in futs]
    finally:
        loop.close()
    assert all(len(r.generated) == 6 for r in done)
    # one forward for the three of them, padded to the next power of two (few graph shapes)
    assert max(len(seqs) for seqs in engine.runner.calls) == 4
    assert GpuRagEngine.decode_bucket(3, 4) == 4 and GpuRagEngine.decode_bucket(5, 6) == 6 and GpuRagEngine.decode_bucket(1, 4) == 1
    assert engine.blocks.num_free == 32


def test_missed_chunks_are_stored_as_computed_alone(engine):
    """``store_misses``: a missed chunk at offset 0 is saved from the request's own blocks; a missed
    chunk behind other context is recomputed alone at position 0 before it is saved, because what
    the request computed for it has attended to the chunks in front of it."""
    from daser_b200.hashing import hash_tokens

    rng = random.Random(2)
    a, b = ([rng.randrange(1000) for _ in range(32)] for _ in range(2))
    engine.generate([a, b], [4, 5], max_new_tokens=1, store_misses=True)
    # a, b and the query are one run of 66 tokens (in pieces of the runner's 64 tokens per forward);
    # then b once more on its own
    assert _computed(engine.runner.calls) == [(0, 64), (64, 2), (0, 32)]
    probe = engine.sched._ipc.lookup_chunks([hash_tokens(a), hash_tokens(b)], "default")
    assert all(m is not None and m["pos_offset"] == 0 for m in probe)
    engine.runner.calls.clear()
    req = engine.generate([b, a], [4, 5], max_new_tokens=1, store_misses=True)
    assert req.restored_chunks == 2 and _computed(engine.runner.calls) == [(64, 2)]
    assert engine.blocks.num_free == 32


def test_decode_batches_run_while_a_starting_request_waits_for_the_drive(engine, monkeypatch):
    """A request whose chunk is still being read does not hold up the requests that are decoding:
    they get a decode step per look at the reads, and the new request starts when the reads are in."""
    rng = random.Random(3)
    a = [rng.randrange(1000) for _ in range(32)]
    engine.store_chunk(a)
    old = engine.submit(RagRequest([], [1, 2, 3], 8))
    engine.step()                                   # its first token; it now decodes
    assert len(old.generated) == 1 and engine.running == [old]
    looks = []

    def reads_done(ticket):
        looks.append(len(old.generated))
        return len(looks) > 3                       # "in flight" for three looks

    monkeypatch.setattr(engine.worker, "reads_done", reads_done)
    engine.runner.calls.clear()
    new = engine.submit(RagRequest([a], [7], 1))
    engine.step()                                   # the new request's step: three decode steps inside it
    assert new.done and new.restored_chunks == 1
    assert looks == [1, 2, 3, 4] and len(old.generated) == 4
    # the three decode forwards of the old request, then the new request's query
    assert _computed(engine.runner.calls) == [(3, 1), (4, 1), (5, 1), (32, 1)]
    engine.interleave_decode = False
    looks.clear()
    engine.submit(RagRequest([a], [7], 1))
    engine.step()
    assert looks == [] and len(old.generated) == 4  # switched off: the step waits for its reads itself
    while engine.has_work():
        engine.step()
    assert engine.blocks.num_free == 32
