"""The unmodified reference service in front of THIS engine.

The reference's REST service drives a remote vLLM through ``/v1/completions`` and a DaseR control
plane through the Unix socket.  Here both of those are this repository's service process (native
CPU engine, vLLM-compatible routes, embedded control plane).  An uploaded document's chunks must
come back as cached, and an ``/infer`` prompt must get them restored behind the system prompt
(which the reference's own stack cannot do: its index only matches prompt prefixes).
"""

import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

import pytest

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
if not os.path.isdir(os.path.join(REF, "daser")):
    pytest.skip("reference not installed under baseline/_ref", allow_module_level=True)
pytest.importorskip("transformers")
pytest.importorskip("tokenizers")
pytestmark = pytest.mark.slow


def _char_tokenizer(path):
    """A tiny local tokenizer (one token per character) saved where AutoTokenizer can load it."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    chars = [chr(c) for c in range(32, 127)] + ["\\n"]
    vocab = {"[UNK]": 0, **{c: i + 1 for i, c in enumerate(chars)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="[UNK]").save_pretrained(path)
    return path


def test_reference_service_uses_this_engine_and_gets_chunk_hits(tmp_path):
    sys.path.insert(0, REF)
    from fastapi.testclient import TestClient

    from daser.service.http_api import ServiceConfig as RefConfig
    from daser.service.http_api import build_service_app as ref_app

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    sock = str(tmp_path / "d.sock")
    cmd = [sys.executable, "-m", "daser_b200.service", "--engine", "native", "--tokenizer", "byte",
           "--store-path", str(tmp_path / "s.store"), "--index-path", str(tmp_path / "s.index"), "--socket-path", sock,
           "--total-slots", "512", "--host", "127.0.0.1", "--port", str(port)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, PYTHONUNBUFFERED="1"))
    base = f"http://127.0.0.1:{port}"
    try:
        t0 = time.time()
        while True:
            assert proc.poll() is None and time.time() - t0 < 40, "engine service did not come up"
            try:
                with urllib.request.urlopen(base + "/health", timeout=2):
                    break
            except OSError:
                time.sleep(0.3)

        def metric(name):
            with urllib.request.urlopen(base + "/metrics", timeout=5) as r:
                for line in r.read().decode().splitlines():
                    if line.startswith(name + " "):
                        return float(line.split()[1])
            return 0.0

        cfg = RefConfig(vllm_base_url=base, model="toy", tokenizer=_char_tokenizer(str(tmp_path / "tok")),
                        socket_path=sock, block_tokens=16, chunk_blocks=2)
        # the reference's default system prompt is 81 characters: the document's chunks sit at an
        # odd offset of the /infer prompt; the scan finds them at any offset and the engine pads
        with TestClient(ref_app(cfg)) as client:
            assert client.get("/health").json()["vllm"] is True
            text = "the quick brown fox jumps over the lazy dog, twice over and then once more for luck"
            r = client.post("/documents", json={"title": "A", "text": text})
            assert r.status_code == 201, r.text
            body = r.json()
            assert body["chunk_count"] == 2 and body["chunk_count_cached"] == 2  # stored by this engine's prefill
            hits0 = metric("daser_connector_chunk_hits")
            r = client.post("/infer", json={"doc_ids": [body["doc_id"]], "task": "why?", "gen_params": {"max_tokens": 3}})
            assert r.status_code == 200, r.text
            out = r.json()
            assert out["completion_tokens"] == 3 and out["prompt_tokens"] > 64
            # both chunks were found behind the system prompt and restored, not recomputed
            assert metric("daser_connector_chunk_hits") - hits0 >= 2
            listing = client.get("/documents").json()
            assert listing[0]["chunk_count_cached"] == 2
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.communicate(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
    assert proc.returncode == 0
