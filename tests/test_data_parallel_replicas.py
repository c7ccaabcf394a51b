"""Data parallelism: several engine replicas attached to ONE control plane and one store file.

The reference's control plane is a multi-client socket server, so replicated engines are
"architecturally free" there (``daser/server/ipc_server.py:99-101``) but never exercised.  Here:
a chunk stored by one replica is restored by another; replicas that store the same chunk at the
same time end up with one copy; replicas serving concurrently agree with a lone engine.
"""

import random
import threading

import pytest
import torch

from conftest import LiveControlPlane
from daser_b200.engine.rag_cpu import CpuRagEngine
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import PRESETS
from daser_b200.position import RopeReencoder


@pytest.fixture
def plane(tmp_path):
    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=512, slot_size=geo.slot_size, num_layers=cfg.num_layers,
                          num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, dtype_bytes=4)
    lp.plane.position = RopeReencoder(cfg.head_dim, cfg.rope_theta)
    lp.start()
    engines = []

    def replica():
        eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)  # same seed: same weights
        engines.append(eng)
        return eng

    yield cfg, lp, replica
    for e in engines:
        e.close()
    lp.stop()


def test_chunk_stored_by_one_replica_is_restored_by_another(plane):
    cfg, lp, replica = plane
    a, b = replica(), replica()
    rng = random.Random(1)
    chunk = [rng.randrange(cfg.vocab_size) for _ in range(64)]
    query = [rng.randrange(cfg.vocab_size) for _ in range(9)]
    cold = b.run_request([], [chunk], query)          # nothing stored: b computes the chunk
    assert cold.restored == [False]
    a.store_chunk(chunk)
    warm = b.run_request([], [chunk], query)          # b restores what a stored
    assert warm.restored == [True]
    torch.testing.assert_close(warm.logits, cold.logits, atol=1e-4, rtol=1e-4)


def test_replicas_storing_the_same_chunk_at_once_keep_one_copy(plane):
    cfg, lp, replica = plane
    engines = [replica() for _ in range(3)]
    rng = random.Random(2)
    chunk = [rng.randrange(cfg.vocab_size) for _ in range(48)]
    start = threading.Barrier(len(engines))
    errors = []

    def store(eng):
        try:
            start.wait(10)
            eng.store_chunk(chunk)
        except Exception as exc:  # a replica that lost the race must skip, not fail
            errors.append(exc)

    threads = [threading.Thread(target=store, args=(e,)) for e in engines]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors
    slots = 48 // cfg.block_tokens
    assert lp.plane.ring.used_slots == slots        # one copy in the ring, whoever won
    res = engines[0].run_request([], [chunk], [1, 2, 3])
    assert res.restored == [True]


def test_replicas_serve_concurrently_and_agree_with_a_lone_engine(plane):
    cfg, lp, replica = plane
    rng = random.Random(3)
    chunks = [[rng.randrange(cfg.vocab_size) for _ in range(32)] for _ in range(6)]
    lone = replica()
    for c in chunks:
        lone.store_chunk(c)
    requests = [([rng.choice(chunks) for _ in range(3)], [rng.randrange(cfg.vocab_size) for _ in range(5)])
                for _ in range(12)]
    want = [lone.generate(c, q, max_new_tokens=3).generated for c, q in requests]
    engines = [replica() for _ in range(3)]
    got = [None] * len(requests)
    errors = []

    def serve(i, eng):
        try:
            for j in range(i, len(requests), len(engines)):
                c, q = requests[j]
                out = eng.generate(c, q, max_new_tokens=3)
                assert out.restored_chunks == 3
                got[j] = out.generated
        except Exception as exc:
            errors.append(exc)

    threads = [threading.Thread(target=serve, args=(i, e)) for i, e in enumerate(engines)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    assert got == want
