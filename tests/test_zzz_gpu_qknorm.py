"""Qwen3-style per-head query / key norm on the CUDA runner against the fp32 PyTorch model.

Runs last (file name) on purpose: the norm lives in a variant of the RoPE + cache-write kernel
that the Llama models never launch."""

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
    plain = LlamaWeights(PRESETS["tiny-gqa"], 1, 0, wf.embed, wf.layers, wf.final_norm, wf.lm_head)
    pool2 = TorchPagedKV(cfg, 64)
    reference_forward(plain, torch.tensor(tokens[:33]), torch.arange(33), pool2, torch.tensor(table), 0, return_logits=False)
    other = reference_forward(plain, torch.tensor(tokens[33:]), torch.arange(33, 40), pool2, torch.tensor(table), 33)[-1]
    assert torch.nn.functional.cosine_similarity(other, want, dim=0).item() < 0.97
