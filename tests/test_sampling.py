"""Temperature sampling (Gumbel-max) on the oracle engine and through the HTTP front end."""

import random

import torch

from conftest import LiveControlPlane
from daser_b200.engine.rag_cpu import CpuRagEngine
from daser_b200.engine.request import RagRequest
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import PRESETS


def test_draws_follow_the_softmax_and_repeat_with_the_seed():
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]])
    temp = 0.7
    eng = CpuRagEngine.__new__(CpuRagEngine)                  # _sample needs no engine state
    counts = torch.zeros(5)
    for seed in range(6000):
        counts[eng._sample(logits, RagRequest([], [1], 4, temperature=temp, seed=seed))] += 1
    want = torch.softmax(logits[0] / temp, 0)
    assert (counts / counts.sum() - want).abs().max().item() < 0.02
    req = RagRequest([], [1], 4, temperature=temp, seed=11)
    assert eng._sample(logits, req) == eng._sample(logits, req)                       # same seed and step
    assert eng._sample(logits, RagRequest([], [1], 4)) == 2                           # temperature 0: greedy
    seen = set()
    for step in range(40):                                                            # steps draw differently
        req.generated = [0] * step
        seen.add(eng._sample(logits, req))
    assert len(seen) > 1


def test_engine_and_http_sampling_are_reproducible_per_seed(tmp_path):
    from fastapi.testclient import TestClient

    from daser_b200.service.http_api import ByteTokenizer, ServiceConfig, build_service_app
    from daser_b200.service.openai_api import mount_openai_routes
    from daser_b200.service.vllm_client import NativeEngineClient

    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)
    try:
        rng = random.Random(0)
        query = [rng.randrange(cfg.vocab_size) for _ in range(12)]
        greedy = eng.generate([], query, max_new_tokens=8).generated
        a = eng.generate([], query, max_new_tokens=8, temperature=1.5, seed=3).generated
        b = eng.generate([], query, max_new_tokens=8, temperature=1.5, seed=3).generated
        c = eng.generate([], query, max_new_tokens=8, temperature=1.5, seed=4).generated
        assert a == b and a != c and a != greedy
        tok = ByteTokenizer()
        client_obj = NativeEngineClient(eng, tok.decode)
        app = build_service_app(ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2),
                                engine_client=client_obj, tokenizer=tok)
        mount_openai_routes(app, client_obj, tok, lp.socket_path, "toy", "default", 16)
        with TestClient(app) as client:
            def post(**kw):
                r = client.post("/v1/completions", json={"prompt": query, "max_tokens": 8, **kw})
                assert r.status_code == 200, r.text
                return r.json()["choices"][0]["token_ids"]

            assert post() == greedy == post(temperature=0)
            assert post(temperature=1.5, seed=3) == a                       # the engine's draw, over HTTP
            assert post(temperature=1.5, seed=3) == post(temperature=1.5, seed=3)
            draws = {tuple(post(temperature=1.5)) for _ in range(4)}        # unseeded: a fresh seed per request
            assert len(draws) > 1
            assert post(temperature=1.5, seed=3, top_k=1) == greedy         # top_k = 1 is greedy whatever the noise
            assert post(temperature=1.5, seed=3, top_p=0.9) == eng.generate(
                [], query, max_new_tokens=8, temperature=1.5, seed=3, top_p=0.9).generated
    finally:
        eng.close()
        lp.stop()


def test_generation_stops_at_stop_tokens_and_reports_why(tmp_path):
    from fastapi.testclient import TestClient

    from daser_b200.service.http_api import ByteTokenizer, ServiceConfig, build_service_app
    from daser_b200.service.openai_api import mount_openai_routes
    from daser_b200.service.vllm_client import NativeEngineClient

    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)
    try:
        query = [3, 1, 4, 1, 5, 9, 2, 6]
        full = eng.generate([], query, max_new_tokens=10)
        assert full.finish_reason == "length" and len(full.generated) == 10
        stop = full.generated[4]
        first = full.generated.index(stop)
        cut = eng.generate([], query, max_new_tokens=10, stop_token_ids=[stop])
        assert cut.finish_reason == "stop" and cut.generated == full.generated[: first + 1]
        assert eng.blocks.num_free == 128
        tok = ByteTokenizer()
        client_obj = NativeEngineClient(eng, tok.decode, eos_token_ids=[stop])      # the "model's" end-of-sequence id
        app = build_service_app(ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2),
                                engine_client=client_obj, tokenizer=tok)
        mount_openai_routes(app, client_obj, tok, lp.socket_path, "toy", "default", 16)
        with TestClient(app) as client:
            body = client.post("/v1/completions", json={"prompt": query, "max_tokens": 10}).json()
            assert body["choices"][0]["finish_reason"] == "stop"
            assert body["choices"][0]["token_ids"] == cut.generated and body["usage"]["completion_tokens"] == first + 1
            body = client.post("/v1/completions", json={"prompt": query, "max_tokens": 10, "ignore_eos": True}).json()
            assert body["choices"][0]["finish_reason"] == "length" and body["choices"][0]["token_ids"] == full.generated
            other = full.generated[1]
            body = client.post("/v1/completions", json={"prompt": query, "max_tokens": 10, "ignore_eos": True,
                                                        "stop_token_ids": [other]}).json()
            assert body["choices"][0]["token_ids"] == full.generated[: full.generated.index(other) + 1]
    finally:
        eng.close()
        lp.stop()


def test_top_k_and_top_p_thresholds():
    from daser_b200.engine.sampling import apply_truncation, sampling_threshold

    torch.manual_seed(0)
    logits = torch.randn(5, 200) * 2
    inv = torch.tensor([1.0, 1.25, 0.0, 2.0, 1.0])
    k = torch.tensor([5, 0, 5, 50, 0])
    p = torch.tensor([1.0, 0.5, 0.5, 0.3, 1.0])
    tau = sampling_threshold(logits, inv, k, p)
    kept = (logits >= tau[:, None]).sum(-1)
    assert int(kept[0]) == 5 and int(kept[2]) == 200 and int(kept[4]) == 200        # top-k; greedy row and plain row untouched
    for row in (1, 3):                                                              # top-p (after top-k): smallest covering set
        order = logits[row].sort(descending=True).values[: int(k[row]) or 200]
        probs = torch.softmax(order * inv[row], 0)
        want = int(((probs.cumsum(0) - probs) < p[row]).sum())
        assert int(kept[row]) == want >= 1
    # a shard masked with the threshold of the whole row keeps exactly its part of the kept set
    shard = logits[:, 50:120].clone()
    apply_truncation(shard, inv, k, p, whole_rows=logits)
    assert torch.equal(torch.isfinite(shard), logits[:, 50:120] >= tau[:, None])


def test_truncated_draws_stay_inside_the_nucleus_and_follow_it():
    logits = torch.tensor([[2.0, 1.5, 1.0, 0.0, -1.0, -3.0]])
    eng = CpuRagEngine.__new__(CpuRagEngine)
    counts = torch.zeros(6)
    for seed in range(4000):
        counts[eng._sample(logits, RagRequest([], [1], 4, temperature=1.0, seed=seed, top_k=3))] += 1
    want = torch.softmax(logits[0, :3], 0)
    assert counts[3:].sum() == 0 and (counts[:3] / counts.sum() - want).abs().max().item() < 0.03
    counts.zero_()
    for seed in range(4000):
        counts[eng._sample(logits, RagRequest([], [1], 4, temperature=1.0, seed=seed, top_p=0.6))] += 1
    # probabilities .42 .26 .16 ...: the first two reach 0.6
    assert counts[2:].sum() == 0 and counts[0] > counts[1] > 0
