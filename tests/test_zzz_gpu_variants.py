"""Kernel variants that the Llama models with greedy decoding never launch: the Qwen3-style per-head
query / key norm inside the RoPE + cache-write kernel, and temperature sampling inside the argmax
kernel.  Runs last (file name) on purpose."""

import random

import pytest
import torch

from daser_b200.models.llama import PRESETS, LayerWeights, LlamaWeights, TorchPagedKV, reference_forward

pytestmark = pytest.mark.gpu


def _fp32_cpu(w: LlamaWeights) -> LlamaWeights:
    layers = [LayerWeights(*(t.float().cpu() for t in (l.input_norm, l.wqkv, l.wo, l.post_norm, l.w_gate_up, l.w_down)),
                           q_norm=l.q_norm.float().cpu(), k_norm=l.k_norm.float().cpu()) for l in w.layers]
    return LlamaWeights(w.cfg, 1, 0, w.embed.float().cpu(), layers, w.final_norm.float().cpu(),
                        w.lm_head.float().cpu(), gate_up_block=w.gate_up_block)


def test_runner_with_qk_norm_matches_reference_forward():
    from daser_b200.engine.runner import GpuModelRunner, make_step_inputs

    cfg = PRESETS["tiny-gqa-qk"]
    w = LlamaWeights.random(cfg, "cuda", torch.bfloat16, seed=3, std=0.05)
    runner = GpuModelRunner(cfg, w, num_blocks=64, max_tokens=64)
    rng = random.Random(0)
    tokens = [rng.randrange(cfg.vocab_size) for _ in range(40)]
    table = [5, 9, 2, 30]
    runner.forward(make_step_inputs([{"tokens": tokens[:33], "start_pos": 0, "block_table": table}], 16, "cuda"))
    logits = runner.logits(make_step_inputs([{"tokens": tokens[33:], "start_pos": 33, "block_table": table}], 16, "cuda"))
    runner.check_status()
    wf = _fp32_cpu(w)
    pool = TorchPagedKV(cfg, 64)
    reference_forward(wf, torch.tensor(tokens[:33]), torch.arange(33), pool, torch.tensor(table), 0, return_logits=False)
    want = reference_forward(wf, torch.tensor(tokens[33:]), torch.arange(33, 40), pool, torch.tensor(table), 33)[-1]
    got = logits.float().cpu()[0]
    cos = torch.nn.functional.cosine_similarity(got, want, dim=0).item()
    assert cos > 0.98, cos
    assert (got - want).abs().max().item() < 0.15 * want.abs().max().item() + 0.05
    # the norm is not a no-op for these weights: the same model without it answers differently
    import dataclasses

    plain = LlamaWeights(dataclasses.replace(cfg, qk_norm=False), 1, 0, wf.embed, wf.layers, wf.final_norm, wf.lm_head)
    pool2 = TorchPagedKV(cfg, 64)
    reference_forward(plain, torch.tensor(tokens[:33]), torch.arange(33), pool2, torch.tensor(table), 0, return_logits=False)
    other = reference_forward(plain, torch.tensor(tokens[33:]), torch.arange(33, 40), pool2, torch.tensor(table), 33)[-1]
    assert torch.nn.functional.cosine_similarity(other, want, dim=0).item() < 0.97


def test_gumbel_max_sampling_kernel_is_exact_across_vocabulary_shards_and_follows_the_softmax():
    """Temperature sampling as an argmax over Gumbel-perturbed logits: the noise depends on (seed,
    global vocabulary index) only, so two shards that exchange their best (value, index) pick what one
    rank holding the whole row picks; over many seeds the picks follow softmax(logits / T)."""
    from daser_b200.ops import elementwise as ew

    torch.manual_seed(0)
    n, rows, temp = 64, 8192, 0.8
    base = torch.randn(n) * 1.5
    logits = base.repeat(rows, 1).to("cuda", torch.float32).contiguous()
    inv = torch.full((rows,), 1.0 / temp, dtype=torch.float32, device="cuda")
    inv[0] = 0.0                                                   # row 0 stays greedy
    seeds = torch.arange(rows, dtype=torch.int64, device="cuda") * 7919 + 13
    val = torch.empty(rows, dtype=torch.float32, device="cuda")
    idx = torch.empty(rows, dtype=torch.int32, device="cuda")
    ew.argmax(logits, val, idx, sampling=(inv, seeds))
    torch.cuda.synchronize()
    assert int(idx[0]) == int(base.argmax())
    # two shards of 32 with their global offsets, combined by the larger perturbed value
    v = [torch.empty_like(val) for _ in range(2)]
    i = [torch.empty_like(idx) for _ in range(2)]
    for s in range(2):
        ew.argmax(logits[:, 32 * s : 32 * (s + 1)].contiguous(), v[s], i[s], index_offset=32 * s, sampling=(inv, seeds))
    torch.cuda.synchronize()
    combined = torch.where(v[1] > v[0], i[1], i[0])
    assert torch.equal(combined, idx)
    freq = torch.bincount(idx[1:].long().cpu(), minlength=n).float() / (rows - 1)
    want = torch.softmax(base / temp, 0)
    assert (freq - want).abs().max().item() < 0.02, (freq - want).abs().max().item()
    # same seeds, same draw; other seeds, another draw
    idx2 = torch.empty_like(idx)
    ew.argmax(logits, val, idx2, sampling=(inv, seeds))
    idx3 = torch.empty_like(idx)
    ew.argmax(logits, val, idx3, sampling=(inv, seeds + 1))
    torch.cuda.synchronize()
    assert torch.equal(idx2, idx) and not torch.equal(idx3, idx)


def test_truncated_sampling_on_the_device():
    """top-k / top-p masking (PyTorch on the device) followed by the Gumbel-max kernel: ``top_k = 1``
    is greedy whatever the noise, and draws never leave the kept set."""
    from daser_b200.engine.sampling import apply_truncation
    from daser_b200.ops import elementwise as ew

    torch.manual_seed(1)
    rows, n = 512, 256
    logits = (torch.randn(rows, n) * 2).to("cuda", torch.float32).contiguous()
    greedy = logits.argmax(-1).to(torch.int32)
    inv = torch.full((rows,), 1.25, dtype=torch.float32, device="cuda")
    seeds = torch.arange(rows, dtype=torch.int64, device="cuda") + 99
    val = torch.empty(rows, dtype=torch.float32, device="cuda")
    idx = torch.empty(rows, dtype=torch.int32, device="cuda")
    one = logits.clone()
    apply_truncation(one, inv, torch.ones(rows, dtype=torch.int64, device="cuda"), torch.ones(rows, device="cuda"))
    ew.argmax(one, val, idx, sampling=(inv, seeds))
    torch.cuda.synchronize()
    assert torch.equal(idx, greedy)
    nucleus = logits.clone()
    apply_truncation(nucleus, inv, torch.full((rows,), 20, dtype=torch.int64, device="cuda"),
                     torch.full((rows,), 0.8, device="cuda"))
    kept = torch.isfinite(nucleus)
    assert int(kept.sum(-1).max()) <= 20 and int(kept.sum(-1).min()) >= 1
    ew.argmax(nucleus, val, idx, sampling=(inv, seeds))
    torch.cuda.synchronize()
    assert bool(kept.gather(1, idx.long()[:, None]).all())


def test_runner_with_fused_epilogues_matches_the_two_kernel_path(monkeypatch):
    """The opt-in fused epilogues (RoPE + KV write behind the QKV projection, SwiGLU under split-K)
    through the whole runner: same hidden states and the same greedy tokens as the default path, for
    a decode-sized step (split-K, the tile's last CTA finishes) and a prefill-sized one (unsplit)."""
    from daser_b200.engine.runner import GpuModelRunner, make_step_inputs
    from daser_b200.ops import gemm

    cfg = PRESETS["tiny-gqa"]
    rng = random.Random(1)
    tokens = [rng.randrange(cfg.vocab_size) for _ in range(200)]
    table = list(range(3, 3 + 14))
    results = {}
    for name, on in (("plain", "0"), ("fused", "1")):
        monkeypatch.setenv("DASER_FUSE_QKV_ROPE", on)
        monkeypatch.setenv("DASER_FUSE_SWIGLU_SPLIT", on)
        w = LlamaWeights.random(cfg, "cuda", torch.bfloat16, seed=3, std=0.05)
        w.interleave_gate_up_(gemm.GATE_UP_BLOCK)
        runner = GpuModelRunner(cfg, w, num_blocks=64, max_tokens=256, use_graphs=False)
        assert runner.fuse_qkv_rope == (on == "1")
        out = []
        for lo, hi in ((0, 150), (150, 199), (199, 200)):
            inp = make_step_inputs([{"tokens": tokens[lo:hi], "start_pos": lo, "block_table": table}], 16, "cuda")
            out.append(int(runner.forward(inp)[0].item()))
            hidden = runner.normed[: hi - lo].float().clone()
        runner.check_status()
        results[name] = (out, hidden, runner.kv_payload.clone())
    assert results["plain"][0] == results["fused"][0]
    a, b = results["plain"][1], results["fused"][1]
    assert (a - b).abs().max().item() <= 0.03 * a.abs().max().item()
    # the pools agree except for rare fp8 rounding flips (split-K sums in another order)
    same = (results["plain"][2] == results["fused"][2]).float().mean().item()
    assert same > 0.97, same
