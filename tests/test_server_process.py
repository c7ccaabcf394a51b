"""The control plane as a real process: start from the command line, talk to it over the
Unix socket, stop it with SIGTERM, start it again and find the state it saved.

Reference behaviour covered: daser/server/__main__.py (signal-driven shutdown that writes the
index, restore at start-up, refusal to load an index written for another geometry is not trusted).
"""

import os
import signal
import subprocess
import sys
import time


from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.hashing import hash_tokens

SLOT = 16 * 1024


def _spawn(tmp_path, *extra):
    sock = str(tmp_path / "d.sock")
    cmd = [sys.executable, "-m", "daser_b200.server", "--store-path", str(tmp_path / "d.store"),
           "--store-size", str(64 * SLOT), "--socket-path", sock, "--index-path", str(tmp_path / "d.index"),
           "--slot-size", str(SLOT), "--block-tokens", "16", "--model-id", "m", *extra]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, PYTHONUNBUFFERED="1"))
    deadline = time.time() + 60
    while time.time() < deadline:
        if os.path.exists(sock):
            try:
                client = IPCClientSync(sock)
                client.stats()
                return proc, client
            except (OSError, RuntimeError):
                pass
        if proc.poll() is not None:
            raise AssertionError("server exited early:\n" + proc.stdout.read())
        time.sleep(0.1)
    proc.kill()
    raise AssertionError("server did not come up")


def _stop(proc, sig=signal.SIGTERM):
    proc.send_signal(sig)
    try:
        out, _ = proc.communicate(timeout=30)
    except subprocess.TimeoutExpired:
        proc.kill()
        raise
    return out


def test_sigterm_saves_and_restart_restores(tmp_path):
    proc, client = _spawn(tmp_path)
    tokens = list(range(48))
    key = hash_tokens(tokens)
    got = client.alloc_chunk(key, len(tokens), "m")
    assert got["num_slots"] == 3
    client.commit_chunk(key)
    client.call({"op": "register_doc", "doc_id": "d1", "title": "t", "token_count": 48, "chunk_keys": [key]})
    client.close()
    out = _stop(proc)
    assert proc.returncode == 0, out
    assert (tmp_path / "d.index").exists()

    proc2, client2 = _spawn(tmp_path)
    try:
        hit = client2.lookup(tokens, "m")
        assert len(hit) == 1 and hit[0]["chunk_key"] == key and hit[0]["start_slot"] == got["start_slot"]
        docs = client2.call({"op": "list_docs"})["docs"]
        assert [d["doc_id"] for d in docs] == ["d1"] and docs[0]["status"] == "ready"
        fresh = client2.alloc_chunk(hash_tokens(list(range(100, 116))), 16, "m")
        assert fresh["start_slot"] == got["start_slot"] + 3  # the ring head came back too
    finally:
        client2.close()
        out2 = _stop(proc2, signal.SIGINT)
    assert proc2.returncode == 0, out2


def test_restart_with_other_geometry_starts_cold(tmp_path):
    """An index written for another slot count is not trusted: warning, empty ring, no stale hits."""
    proc, client = _spawn(tmp_path)
    toks = list(range(16))
    client.alloc_chunk(hash_tokens(toks), 16, "m")
    client.commit_chunk(hash_tokens(toks))
    client.close()
    _stop(proc)
    proc2, client2 = _spawn(tmp_path, "--slot-size", str(2 * SLOT))  # later flag wins: 32 slots instead of 64
    try:
        assert client2.lookup(toks, "m") == []
        assert client2.stats()["ring"]["used_slots"] == 0
    finally:
        client2.close()
        out = _stop(proc2)
    assert "cold start" in out


def test_periodic_snapshot_survives_sigkill(tmp_path):
    proc, client = _spawn(tmp_path, "--snapshot-interval", "0.2")
    client.alloc_chunk(hash_tokens(list(range(32))), 32, "m")
    client.commit_chunk(hash_tokens(list(range(32))))
    client.close()
    deadline = time.time() + 20
    while not (tmp_path / "d.index").exists() and time.time() < deadline:
        time.sleep(0.1)
    time.sleep(0.5)
    proc.kill()  # no chance to save on the way out
    proc.wait(timeout=30)
    proc2, client2 = _spawn(tmp_path)
    try:
        assert len(client2.lookup(list(range(32)), "m")) == 1
    finally:
        client2.close()
        _stop(proc2)


def test_service_process_with_batching_serves_concurrent_clients(tmp_path):
    """`--native-batching`: the engine loop behind the HTTP front end.  Eight clients at once get
    the answers a lone client gets, the process shuts down cleanly with the loop drained."""
    import json
    import socket
    import urllib.request
    from concurrent.futures import ThreadPoolExecutor

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "daser_b200.service", "--engine", "native", "--native-batching", "--tokenizer", "byte",
           "--store-path", str(tmp_path / "s.store"), "--index-path", str(tmp_path / "s.index"),
           "--socket-path", str(tmp_path / "s.sock"), "--total-slots", "256", "--host", "127.0.0.1", "--port", str(port)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, PYTHONUNBUFFERED="1"))
    base = f"http://127.0.0.1:{port}"

    def post(prompt):
        body = json.dumps({"prompt": prompt, "max_tokens": 4}).encode()
        req = urllib.request.Request(base + "/v1/completions", data=body, headers={"content-type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            return json.load(r)["choices"][0]["token_ids"]

    try:
        t0 = time.time()
        while True:
            assert proc.poll() is None, "service exited early"
            assert time.time() - t0 < 25, "service did not come up within 25 s"
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    if json.load(r)["status"] == "ok":
                        break
            except OSError:
                time.sleep(0.3)
        prompts = [[(3 * i + j) % 200 + 1 for j in range(24 + i)] for i in range(8)]
        with ThreadPoolExecutor(8) as pool:
            together = list(pool.map(post, prompts))
        assert together == [post(p) for p in prompts] and all(len(t) == 4 for t in together)
        with urllib.request.urlopen(base + "/metrics", timeout=5) as r:
            assert "daser_engine_loop_in_flight" in r.read().decode()
    finally:
        out_text = _stop(proc)
    assert proc.returncode == 0, out_text[-2000:]


def test_service_process_with_native_engine_starts_quickly_and_answers(tmp_path):
    """`python -m daser_b200.service --engine native`: control plane, CPU engine and REST front end
    in one process.  The engine is built off the event loop (its connector talks to the control
    plane that the same loop serves), so start-up must not wait for an RPC timeout."""
    import json
    import socket
    import urllib.request

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "daser_b200.service", "--engine", "native", "--tokenizer", "byte",
           "--store-path", str(tmp_path / "s.store"), "--index-path", str(tmp_path / "s.index"),
           "--socket-path", str(tmp_path / "s.sock"), "--total-slots", "256", "--host", "127.0.0.1", "--port", str(port)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, PYTHONUNBUFFERED="1"))
    base = f"http://127.0.0.1:{port}"
    try:
        t0 = time.time()
        up = False
        while time.time() - t0 < 25:
            if proc.poll() is not None:
                raise AssertionError("service exited early:\n" + proc.stdout.read())
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    up = json.load(r)["status"] == "ok"
                    break
            except OSError:
                time.sleep(0.3)
        assert up, "service did not come up within 25 s"
        body = json.dumps({"prompt": "what does the fox say? nobody knows for sure", "max_tokens": 2}).encode()
        req = urllib.request.Request(base + "/v1/completions", data=body, headers={"content-type": "application/json"})
        with urllib.request.urlopen(req, timeout=30) as r:
            out = json.load(r)
        assert out["usage"]["completion_tokens"] == 2 and out["object"] == "text_completion"

        # this repository's client for a remote vLLM, pointed at the native engine instead
        import asyncio

        from daser_b200.service.vllm_client import VLLMClient

        async def through_the_vllm_client():
            async with VLLMClient(base, "toy") as c:
                assert await c.health()
                chunk = list(range(10, 42))
                await c.prefill(chunk)  # max_tokens = 1: leaves the chunk in the store
                prompt = [5] * 16 + chunk + [7, 8, 9]
                reply = await c.completion(prompt, {"max_tokens": 2, "temperature": 0})
                streamed = [item async for item in c.completion_stream(prompt, {"max_tokens": 2, "temperature": 0})]
                return reply, streamed

        reply, streamed = asyncio.run(through_the_vllm_client())
        usage = reply["usage"]
        assert usage["completion_tokens"] == 2 and usage["prompt_tokens"] == 51
        # the same request over server-sent events: token by token, the same tokens, usage at the end
        assert [t for item in streamed[:-1] for t in item["token_ids"]] == reply["choices"][0]["token_ids"]
        assert len(streamed) == 3 and streamed[-1] == {"done": True, "usage": usage}
        with urllib.request.urlopen(base + "/metrics", timeout=5) as r:
            text = r.read().decode()
        hits = [float(l.split()[1]) for l in text.splitlines() if l.startswith("daser_connector_chunk_hits ")]
        assert hits and hits[0] >= 1  # the prefilled chunk was found behind the 16-token lead and restored
    finally:
        out_text = _stop(proc)
    assert proc.returncode == 0, out_text[-2000:]
    assert (tmp_path / "s.index").exists()  # state saved on the way out


def test_operator_cli_reads_and_evicts(tmp_path, capsys):
    import json

    from daser_b200.server import ctl

    proc, client = _spawn(tmp_path)
    try:
        key = hash_tokens(list(range(32)))
        client.alloc_chunk(key, 32, "m")
        client.commit_chunk(key)
        sock = str(tmp_path / "d.sock")
        assert ctl.main(["--socket-path", sock, "stats"]) == 0
        assert json.loads(capsys.readouterr().out)["ring"]["used_slots"] == 2
        assert ctl.main(["--socket-path", sock, "lookup", key, "nope", "--model-id", "m"]) == 0
        found = json.loads(capsys.readouterr().out)["chunks"]
        assert found[0]["chunk_key"] == key and found[1] is None
        assert ctl.main(["--socket-path", sock, "evict-chunk", key]) == 0
        capsys.readouterr()
        assert ctl.main(["--socket-path", sock, "lookup", key, "--model-id", "m"]) == 0
        assert json.loads(capsys.readouterr().out)["chunks"] == [None]
        assert "tokens_bin" in json.loads((ctl.main(["--socket-path", sock, "hello"]), capsys.readouterr().out)[1])["features"]
        assert ctl.main(["--socket-path", sock, "doc", "missing"]) == 1  # server-side error -> exit code 1
        assert ctl.main(["--socket-path", str(tmp_path / "absent.sock"), "--timeout", "1", "stats"]) == 1
    finally:
        client.close()
        _stop(proc)
