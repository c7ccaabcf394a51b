"""REST service over a live control plane, with a fake engine and with the CPU engine."""

import asyncio

import pytest
from fastapi.testclient import TestClient

from conftest import LiveControlPlane
from daser_b200.hashing import hash_tokens
from daser_b200.service.chunker import Chunker
from daser_b200.service.http_api import ByteTokenizer, ServiceConfig, build_service_app


class FakeEngine:
    """Stands in for vLLM: 'prefill' stores nothing, so chunks count as not cached."""

    def __init__(self, plane=None, up=True):
        self.prefills, self.completions, self.up, self.fail = [], [], up, False
        self.plane = plane

    @property
    def model(self):
        return "fake"

    async def close(self):
        pass

    async def health(self):
        return self.up

    async def prefill(self, tokens):
        if self.fail:
            raise RuntimeError("engine down")
        self.prefills.append(list(tokens))
        if self.plane is not None:  # emulate the connector's store + commit
            from daser_b200.connector.ipc_client import IPCClientSync

            c = IPCClientSync(self.plane.socket_path)
            key = hash_tokens(list(tokens))
            await asyncio.get_running_loop().run_in_executor(None, c.alloc_chunk, key, len(tokens), "default")
            await asyncio.get_running_loop().run_in_executor(None, c.commit_chunk, key)
            c.close()

    async def completion(self, tokens, gen_params=None, segments=None):
        if self.fail:
            raise RuntimeError("engine down")
        self.completions.append((list(tokens), gen_params, segments))
        return {"choices": [{"text": "answer"}], "usage": {"prompt_tokens": len(tokens), "completion_tokens": 3}}


def test_chunker():
    ch = Chunker(4, 2)
    toks = list(range(19))
    chunks = ch.chunk(toks)
    assert [c.tokens for c in chunks] == [toks[0:8], toks[8:16]]  # trailing 3 dropped
    assert chunks[1].chunk_key == hash_tokens(toks[8:16]) and ch.tail(toks) == toks[16:]
    assert ch.chunk_tokens == 8 and ch.chunk(list(range(5))) == []
    with pytest.raises(ValueError):
        Chunker(0, 1)


@pytest.fixture
def svc(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    eng = FakeEngine(lp)
    cfg = ServiceConfig("http://unused", "fake", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2)
    app = build_service_app(cfg, engine_client=eng, tokenizer=ByteTokenizer())
    with TestClient(app) as client:
        yield client, eng
    lp.stop()


def test_document_lifecycle_and_infer(svc):
    client, eng = svc
    assert client.get("/health").json() == {"status": "ok", "vllm": True}
    assert client.post("/documents", json={"title": "t", "text": "short"}).status_code == 400
    text = "The quick brown fox jumps over the lazy dog. " * 3  # 135 bytes -> 4 chunks of 32
    r = client.post("/documents", json={"title": "Doc A", "text": text})
    assert r.status_code == 201
    body = r.json()
    assert body["status"] == "ready" and body["chunk_count"] == 4 and body["chunk_count_cached"] == 4
    assert len(eng.prefills) == 4 and body["prefill_ms"] >= 0
    doc_id = body["doc_id"]
    listing = client.get("/documents").json()
    assert listing[0]["doc_id"] == doc_id and listing[0]["chunk_count_total"] == 4
    doc = client.get(f"/documents/{doc_id}").json()
    assert "tokens" not in doc and doc["cached_mask"] == [True] * 4
    assert client.get("/documents/nope").status_code == 404
    assert client.post("/infer", json={"doc_ids": [], "task": "x"}).status_code == 400
    assert client.post("/infer", json={"doc_ids": ["nope"], "task": "x"}).status_code == 404
    r = client.post("/infer", json={"doc_ids": [doc_id], "task": "Summarise", "gen_params": {"max_tokens": 5}})
    assert r.status_code == 200
    out = r.json()
    assert out["text"] == "answer" and out["completion_tokens"] == 3 and out["latency_ms"] >= 0
    prompt, params, segments = eng.completions[-1]
    assert params == {"max_tokens": 5}
    assert [t for s in segments for t in s] == prompt
    # the document's chunks appear as their own segments, so the engine can look them up by key
    keys = {hash_tokens(s) for s in segments}
    assert set(doc["chunk_keys"]) <= keys
    assert "daser_ipc_register_doc" in client.get("/metrics").text
    assert client.delete(f"/documents/{doc_id}").json() == {"ok": True, "chunks_evicted": 4}
    assert client.delete(f"/documents/{doc_id}").status_code == 404
    assert client.get("/documents").json() == []


def test_engine_failures_map_to_502_and_health_degrades(svc):
    client, eng = svc
    eng.up = False
    assert client.get("/health").json() == {"status": "degraded", "vllm": False}
    text = "".join(chr(97 + (i * 7) % 26) for i in range(100))  # three distinct 32-byte chunks
    eng.fail = True
    assert client.post("/documents", json={"title": "t", "text": text}).status_code == 502
    eng.fail = False
    r = client.post("/documents", json={"title": "t", "text": text})
    assert r.status_code == 201, r.text
    doc_id = r.json()["doc_id"]
    eng.fail = True
    assert client.post("/infer", json={"doc_ids": [doc_id], "task": "q"}).status_code == 502


def test_service_cli_flags():
    from daser_b200.service.__main__ import _build_daser_config, _parse_args

    a = _parse_args(["--vllm-base-url", "http://x", "--model", "m", "--tokenizer", "byte"])
    assert (a.host, a.port, a.total_slots, a.slot_size, a.chunk_blocks) == ("0.0.0.0", 8080, 1024, 0, 16)
    assert a.store_path == "/mnt/xfs/daser.store" and a.index_path == "/mnt/xfs/daser.index"
    cfg = _build_daser_config(a)
    assert cfg.total_slots == 1024 and cfg.slot_size == 0
    with pytest.raises(SystemExit):
        _parse_args(["--tokenizer", "byte"])  # vllm engine needs url + model
    assert _parse_args(["--engine", "native", "--tokenizer", "byte"]).native_model == "toy"


def test_native_cpu_engine_serves_infer_with_restored_chunks(tmp_path):
    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.kv.layout import KVGeometry
    from daser_b200.models.llama import PRESETS
    from daser_b200.service.vllm_client import NativeEngineClient
    from daser_b200 import metrics

    mcfg = PRESETS["toy"]
    geo = KVGeometry(mcfg.num_layers, mcfg.num_kv_heads, mcfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    engine = CpuRagEngine(mcfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)
    tok = ByteTokenizer()
    client_obj = NativeEngineClient(engine, tok.decode)
    cfg = ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2)
    app = build_service_app(cfg, engine_client=client_obj, tokenizer=tok)
    try:
        with TestClient(app) as client:
            doc_id = client.post("/documents", json={"title": "A", "text": "lorem ipsum dolor sit amet " * 5}).json()["doc_id"]
            hits0 = metrics.snapshot().get("connector.chunk_hits", 0)
            r = client.post("/infer", json={"doc_ids": [doc_id], "task": "why?", "gen_params": {"max_tokens": 1}})
            assert r.status_code == 200 and r.json()["completion_tokens"] == 1
            # uploaded chunks were found and restored inside a prompt that starts with the system prompt
            assert metrics.snapshot().get("connector.chunk_hits", 0) - hits0 >= 4
    finally:
        engine.close()
        lp.stop()


def test_native_client_degrades_after_a_lost_peer():
    """A step that ends with PeerLost marks the in-process engine unavailable: health turns false
    and later calls fail at once instead of launching work that would wait for the dead rank."""
    import asyncio

    from daser_b200.parallel.health import PeerLost
    from daser_b200.service.vllm_client import NativeEngineClient

    class Engine:
        class cfg:
            block_tokens = 16

        calls = 0

        def generate(self, chunks, query, max_new_tokens=1):
            Engine.calls += 1
            raise PeerLost([3], "left the group")

    client = NativeEngineClient(Engine(), lambda ids: "")

    async def run():
        assert await client.health()
        for _ in range(2):
            try:
                await client.completion([1, 2, 3], {"max_tokens": 1})
            except RuntimeError:
                pass
        return await client.health()

    assert asyncio.run(run()) is False
    assert Engine.calls == 1


def test_split_at_hits():
    from daser_b200.service.openai_api import split_at_hits

    toks = list(range(100))
    hits = [{"offset": 32, "token_count": 32}, {"offset": 16, "token_count": 32},  # the second overlaps: dropped
            {"offset": 80, "token_count": 20}]                                      # would leave no query: dropped
    segs = split_at_hits(toks, hits, 16)
    assert segs == [toks[0:16], toks[16:48], toks[48:]]
    odd = [{"offset": 21, "token_count": 32}]
    assert split_at_hits(toks, odd, 16) == [toks[:21], toks[21:53], toks[53:]]  # the engine client pads the gap
    assert split_at_hits(toks, odd, 16, aligned_only=True) == [toks]
    assert split_at_hits(toks, [], 16) == [toks]
    assert [t for s in segs for t in s] == toks and segs[-1]


def test_openai_completions_reuse_stored_chunks_found_by_scan(tmp_path):
    """The native engine behind vLLM's completions API: a prompt that contains an uploaded chunk
    behind an unrelated prefix gets it restored, and the reference's kind of client (token-id
    prompt, max_tokens) gets the usual response shape."""
    from daser_b200 import metrics
    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.kv.layout import KVGeometry
    from daser_b200.models.llama import PRESETS
    from daser_b200.service.openai_api import mount_openai_routes
    from daser_b200.service.vllm_client import NativeEngineClient

    mcfg = PRESETS["toy"]
    geo = KVGeometry(mcfg.num_layers, mcfg.num_kv_heads, mcfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    engine = CpuRagEngine(mcfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)
    tok = ByteTokenizer()
    client_obj = NativeEngineClient(engine, tok.decode)
    cfg = ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2)
    app = build_service_app(cfg, engine_client=client_obj, tokenizer=tok)
    mount_openai_routes(app, client_obj, tok, lp.socket_path, "toy", "default", 16)
    try:
        with TestClient(app) as client:
            text = "the quick brown fox jumps over the lazy dog and keeps running "  # 62 bytes -> one 32-token chunk
            assert client.post("/documents", json={"title": "A", "text": text}).status_code == 201
            enc = lambda t: tok(t)["input_ids"]  # noqa: E731
            chunk = enc(text)[:32]
            prompt = list(range(1, 17)) + chunk + enc("and then?")
            assert client.get("/v1/models").json()["data"][0]["id"] == "toy"
            hits0 = metrics.snapshot().get("connector.chunk_hits", 0)
            r = client.post("/v1/completions", json={"model": "toy", "prompt": prompt, "max_tokens": 3, "temperature": 0})
            assert r.status_code == 200, r.text
            body = r.json()
            assert body["object"] == "text_completion" and len(body["choices"][0]["token_ids"]) == 3
            assert body["usage"] == {"prompt_tokens": len(prompt), "completion_tokens": 3, "total_tokens": len(prompt) + 3}
            assert metrics.snapshot().get("connector.chunk_hits", 0) - hits0 >= 1  # the chunk was restored, not recomputed
            # the same prompt with nothing cached computes the same first token
            cold = client.post("/v1/completions", json={"prompt": [7] * 16 + prompt[16:], "max_tokens": 1})
            assert cold.status_code == 200
            # bad requests
            assert client.post("/v1/completions", json={"prompt": [], "max_tokens": 1}).status_code == 400
            assert client.post("/v1/completions", json={"prompt": prompt, "max_tokens": 0}).status_code == 400
            # streaming: one event per token, the same tokens as the plain call, usage at the end
            with client.stream("POST", "/v1/completions", json={"prompt": prompt, "max_tokens": 3, "stream": True}) as sr:
                assert sr.status_code == 200 and sr.headers["content-type"].startswith("text/event-stream")
                events = [line[6:] for line in sr.iter_lines() if line.startswith("data: ")]
            assert events[-1] == "[DONE]"
            import json as _json

            objs = [_json.loads(e) for e in events[:-1]]
            streamed = [t for o in objs for t in o["choices"][0]["token_ids"]]
            assert streamed == body["choices"][0]["token_ids"]
            assert [len(o["choices"][0]["token_ids"]) for o in objs] == [1, 1, 1, 0]
            assert "".join(o["choices"][0]["text"] for o in objs) == body["choices"][0]["text"]
            assert objs[-1]["choices"][0]["finish_reason"] == "length" and objs[-1]["usage"] == body["usage"]
            assert metrics.snapshot().get("service.stream_ttft_ms.count", 0) >= 1
            assert client.post("/v1/completions", json={"prompt": "plain text works too", "max_tokens": 1}).status_code == 200
    finally:
        engine.close()
        lp.stop()


def test_batching_engine_client_serves_concurrent_and_streamed_requests(tmp_path):
    """With ``batching`` the engine client hands requests to an engine loop: concurrent HTTP calls share
    the engine's steps, answers equal those of the one-at-a-time client, streaming still works."""
    import json
    from concurrent.futures import ThreadPoolExecutor

    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.kv.layout import KVGeometry
    from daser_b200.models.llama import PRESETS
    from daser_b200.service.openai_api import mount_openai_routes
    from daser_b200.service.vllm_client import NativeEngineClient

    mcfg = PRESETS["toy"]
    geo = KVGeometry(mcfg.num_layers, mcfg.num_kv_heads, mcfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    engine = CpuRagEngine(mcfg, lp.socket_path, lp.cfg.store_path, num_blocks=256)
    tok = ByteTokenizer()
    client_obj = NativeEngineClient(engine, tok.decode, batching=True)
    cfg = ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2)
    app = build_service_app(cfg, engine_client=client_obj, tokenizer=tok)
    mount_openai_routes(app, client_obj, tok, lp.socket_path, "toy", "default", 16)
    prompts = [[(7 * i + j) % 250 + 1 for j in range(20 + i)] for i in range(6)]
    try:
        with TestClient(app) as client:
            assert client.post("/documents", json={"title": "A", "text": "lorem ipsum dolor sit amet " * 5}).status_code == 201
            post = lambda p: client.post("/v1/completions", json={"prompt": p, "max_tokens": 6}).json()  # noqa: E731
            with ThreadPoolExecutor(6) as pool:
                together = list(pool.map(post, prompts))
            alone = [post(p) for p in prompts]
            assert [r["choices"][0]["token_ids"] for r in together] == [r["choices"][0]["token_ids"] for r in alone]
            assert client_obj._loop.max_batch > 1
            # several prompts in one call: one choice per prompt, in order, usage summed
            many = client.post("/v1/completions", json={"prompt": prompts[:3], "max_tokens": 6}).json()
            assert [c["index"] for c in many["choices"]] == [0, 1, 2]
            assert [c["token_ids"] for c in many["choices"]] == [r["choices"][0]["token_ids"] for r in alone[:3]]
            assert many["usage"]["completion_tokens"] == 18
            assert many["usage"]["prompt_tokens"] == sum(len(p) for p in prompts[:3])
            assert client.post("/v1/completions", json={"prompt": prompts[:2], "stream": True}).status_code == 400
            with client.stream("POST", "/v1/completions", json={"prompt": prompts[0], "max_tokens": 6, "stream": True}) as sr:
                events = [json.loads(l[6:]) for l in sr.iter_lines() if l.startswith("data: {")]
            assert [t for e in events for t in e["choices"][0]["token_ids"]] == alone[0]["choices"][0]["token_ids"]
            assert client.get("/health").json()["status"] in ("ok", "healthy", "degraded")
    finally:
        import asyncio

        asyncio.run(client_obj.close())
        engine.close()
        lp.stop()


def test_chat_completions_route(tmp_path):
    import json

    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.kv.layout import KVGeometry
    from daser_b200.models.llama import PRESETS
    from daser_b200.service.openai_api import chat_prompt_tokens, mount_openai_routes
    from daser_b200.service.vllm_client import NativeEngineClient

    mcfg = PRESETS["toy"]
    geo = KVGeometry(mcfg.num_layers, mcfg.num_kv_heads, mcfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=128, slot_size=geo.slot_size).start()
    engine = CpuRagEngine(mcfg, lp.socket_path, lp.cfg.store_path, num_blocks=128)
    tok = ByteTokenizer()
    client_obj = NativeEngineClient(engine, tok.decode)
    app = build_service_app(ServiceConfig("", "toy", "byte", lp.socket_path, block_tokens=16, chunk_blocks=2),
                            engine_client=client_obj, tokenizer=tok)
    mount_openai_routes(app, client_obj, tok, lp.socket_path, "toy", "default", 16)
    messages = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "why is the sky blue?"}]
    try:
        with TestClient(app) as client:
            ids = chat_prompt_tokens(tok, messages)
            assert tok.decode(ids) == "system: be brief\nuser: why is the sky blue?\nassistant:"
            plain = client.post("/v1/completions", json={"prompt": ids, "max_tokens": 4}).json()
            r = client.post("/v1/chat/completions", json={"model": "toy", "messages": messages, "max_tokens": 4})
            assert r.status_code == 200, r.text
            body = r.json()
            assert body["object"] == "chat.completion" and body["id"].startswith("chatcmpl-")
            msg = body["choices"][0]["message"]
            assert msg["role"] == "assistant" and msg["content"] == plain["choices"][0]["text"]
            assert body["usage"]["prompt_tokens"] == len(ids) and body["usage"]["completion_tokens"] == 4
            with client.stream("POST", "/v1/chat/completions",
                               json={"messages": messages, "max_tokens": 4, "stream": True}) as sr:
                events = [json.loads(l[6:]) for l in sr.iter_lines() if l.startswith("data: {")]
            assert all(e["object"] == "chat.completion.chunk" for e in events)
            assert "".join(e["choices"][0]["delta"]["content"] for e in events) == msg["content"]
            assert events[-1]["choices"][0]["finish_reason"] == "length"
            assert client.post("/v1/chat/completions", json={"messages": [], "max_tokens": 1}).status_code == 400
            for unsupported in ({"n": 2}, {"best_of": 3}, {"logprobs": 5}, {"echo": True}, {"stop": ["\n\n"]}):
                r = client.post("/v1/completions", json={"prompt": ids, "max_tokens": 1, **unsupported})
                assert r.status_code == 400 and "not supported" in r.json()["detail"]
            assert client.post("/v1/completions", json={"prompt": ids, "max_tokens": 1, "n": 1, "top_p": 0.9}).status_code == 200
    finally:
        engine.close()
        lp.stop()


def test_abandoned_stream_keeps_the_lock_until_the_engine_is_through(tmp_path):
    """Without the engine loop one worker thread at a time owns the engine: a consumer that stops
    reading must not let the next request in while that thread is still generating."""
    import threading
    import time

    from daser_b200.service.vllm_client import NativeEngineClient

    class SlowEngine:
        class cfg:
            block_tokens = 16

        def __init__(self):
            self.inside = 0
            self.overlap = False

        def generate(self, chunks, query, max_new_tokens=1, on_token=None, **kw):
            self.inside += 1
            self.overlap = self.overlap or self.inside > 1
            out = []
            for i in range(max_new_tokens):
                time.sleep(0.01)
                out.append(65 + i % 26)
                if on_token:
                    on_token(out[-1])
            self.inside -= 1
            return type("R", (), {"generated": out, "context_len": len(query), "finish_reason": "length"})()

    eng = SlowEngine()
    client = NativeEngineClient(eng, lambda ids: "".join(map(chr, ids)))

    async def scenario():
        agen = client.completion_stream([1, 2, 3], {"max_tokens": 30})
        async for _ in agen:
            break                                              # the consumer goes away after one token
        closing = asyncio.ensure_future(agen.aclose())
        nxt = await client.completion([4, 5], {"max_tokens": 3})   # must wait for the first to end
        await closing
        return nxt

    out = asyncio.run(scenario())
    assert out["choices"][0]["token_ids"] == [65, 66, 67] and not eng.overlap and threading.active_count() >= 1
