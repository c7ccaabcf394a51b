"""Checkpoints in the Hugging Face layout, and this package's model against ``transformers``' own
implementation of the same architectures (small random models, CPU, fp32)."""

import pytest
import torch

from daser_b200.models import hf
from daser_b200.models.llama import TorchPagedKV, reference_forward, shard_weights

transformers = pytest.importorskip("transformers")


def _logits(weights, ids):
    cfg = weights.cfg
    pool = TorchPagedKV(cfg, -(-len(ids) // cfg.block_tokens) + 1)
    table = torch.arange(pool.num_blocks)
    # in two pieces, so that the second attends to a cached first (the serving pattern)
    cut = len(ids) // 2
    first = reference_forward(weights, torch.tensor(ids[:cut]), torch.arange(cut), pool, table, 0)
    second = reference_forward(weights, torch.tensor(ids[cut:]), torch.arange(cut, len(ids)), pool, table, cut)
    return torch.cat([first, second])


def _tiny_llama(vocab=97, **kw):
    cfg = transformers.LlamaConfig(
        vocab_size=vocab, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=500000.0,
        tie_word_embeddings=False, attention_bias=False, mlp_bias=False, **kw)
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).eval()


def test_llama_matches_transformers_including_llama3_rope_scaling():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 32}
    for kw in ({}, {"rope_scaling": scaling}):
        model = _tiny_llama(**kw)
        cfg = hf.config_from_hf(model.config)
        assert (cfg.hidden, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate) == (64, 4, 2, 16, 160)
        assert bool(cfg.rope_scaling) == bool(kw) and not cfg.qk_norm
        w = hf.weights_from_state_dict(cfg, model.state_dict(), dtype=torch.float32)
        ids = [(7 * i * i + 3) % 97 for i in range(90)]           # positions well past the scaled wavelengths
        with torch.no_grad():
            want = model(torch.tensor([ids])).logits[0]
        got = _logits(w, ids)
        assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item()), kw


def test_qwen3_matches_transformers():
    cfg_hf = transformers.Qwen3Config(
        vocab_size=101, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(1)
    model = transformers.Qwen3ForCausalLM(cfg_hf).eval()
    with torch.no_grad():                                        # norms are initialised to one: perturb them
        for name, p in model.named_parameters():
            if name.endswith("norm.weight"):
                p.add_(0.2 * torch.randn_like(p))
    cfg = hf.config_from_hf(model.config)
    assert cfg.qk_norm and cfg.head_dim == 32 and cfg.num_heads * cfg.head_dim != cfg.hidden
    w = hf.weights_from_state_dict(cfg, model.state_dict(), dtype=torch.float32)
    ids = [(5 * i + 11) % 101 for i in range(50)]
    with torch.no_grad():
        want = model(torch.tensor([ids])).logits[0]
    got = _logits(w, ids)
    assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())


def test_checkpoint_directory_loads_per_rank_and_round_trips(tmp_path):
    model = _tiny_llama(vocab=96)
    model.save_pretrained(tmp_path / "ckpt", safe_serialization=True, max_shard_size="40KB")   # several shards
    assert (tmp_path / "ckpt" / "model.safetensors.index.json").exists()
    full = hf.load_checkpoint(str(tmp_path / "ckpt"), dtype=torch.float32)
    assert full.cfg.num_layers == 2 and full.meta["tied_head"] is False
    for rank in range(2):
        mine = hf.load_checkpoint(str(tmp_path / "ckpt"), tp=2, rank=rank, dtype=torch.float32)
        want = shard_weights(full, 2, rank)
        assert torch.equal(mine.lm_head, want.lm_head) and torch.equal(mine.embed, want.embed)
        for a, b in zip(mine.layers, want.layers):
            for f in ("wqkv", "wo", "w_gate_up", "w_down", "input_norm", "post_norm"):
                assert torch.equal(getattr(a, f), getattr(b, f)), (rank, f)
    back = hf.state_dict_of(full)
    sd = model.state_dict()
    assert set(back) == {k for k in sd if "rotary" not in k}
    assert all(torch.equal(back[k], sd[k]) for k in back)
    # a checkpoint with tied embeddings has no lm_head: the output projection is the embedding
    tied_sd = {k: v for k, v in sd.items() if k != "lm_head.weight"}
    tied = hf.weights_from_state_dict(full.cfg, tied_sd, dtype=torch.float32)
    assert tied.meta["tied_head"] and torch.equal(tied.lm_head, tied.embed)
    with pytest.raises(ValueError):
        hf.config_from_hf({"model_type": "gpt2"})


def test_service_process_serves_a_checkpoint_and_agrees_with_transformers_greedy(tmp_path):
    """`python -m daser_b200.service --engine native --native-checkpoint <dir>`: the tokens that come
    back over HTTP are the ones `transformers` generates greedily from the same checkpoint, on the
    first call (all computed, block-aligned prefix stored) and on the second (prefix restored)."""
    import json
    import os
    import signal
    import socket
    import subprocess
    import sys
    import time
    import urllib.request

    model = _tiny_llama(vocab=320)
    model.save_pretrained(tmp_path / "ckpt", safe_serialization=True)
    prompt = [(11 * i + 5) % 256 for i in range(45)]
    with torch.no_grad():
        want = model.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False)[0, len(prompt):].tolist()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "daser_b200.service", "--engine", "native", "--native-checkpoint", str(tmp_path / "ckpt"),
           "--tokenizer", "byte", "--store-path", str(tmp_path / "s.store"), "--index-path", str(tmp_path / "s.index"),
           "--socket-path", str(tmp_path / "s.sock"), "--total-slots", "128", "--host", "127.0.0.1", "--port", str(port)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, PYTHONUNBUFFERED="1"))
    base = f"http://127.0.0.1:{port}"

    def post(body):
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps(body).encode(),
                                     headers={"content-type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            return json.load(r)

    try:
        t0 = time.time()
        while True:
            assert proc.poll() is None, "service exited early:\n" + (proc.stdout.read() if proc.stdout else "")
            assert time.time() - t0 < 40, "service did not come up"
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    if json.load(r)["status"] == "ok":
                        break
            except OSError:
                time.sleep(0.3)
        post({"prompt": prompt[:32], "max_tokens": 1})                   # stores the 32-token prefix
        cold = post({"prompt": prompt, "max_tokens": 6})["choices"][0]["token_ids"]
        with urllib.request.urlopen(base + "/metrics", timeout=5) as r:
            text = r.read().decode()
        hits = [float(l.split()[1]) for l in text.splitlines() if l.startswith("daser_connector_chunk_hits ")]
        assert cold == want
        assert hits and hits[0] >= 1                                     # the second call restored the prefix
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(30)
        except subprocess.TimeoutExpired:
            proc.kill()
    assert proc.returncode == 0
