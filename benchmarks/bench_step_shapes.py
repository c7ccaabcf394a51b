"""How long does ONE rank's share of a tensor-parallel step take when nothing has to be exchanged?

    python benchmarks/bench_step_shapes.py [--tp 1,2,4,8] [--tokens 64] [--ctx 3328] [--iters 20]

For each degree the Llama-3-70B layer is cut as tensor parallelism cuts it (heads, KV heads,
intermediate size and vocabulary divided by tp; hidden size and layer count unchanged) and that
shard runs ALONE on one GPU as if it were a whole model: same kernels, same CUDA graphs, no peer,
no flag, no reduction.  The figure is the floor of the multi-GPU step's compute part: what is left
between it and the measured step of `bench_tp_forms.py` is what the exchange costs.  With
`--launches` the last step is repeated eagerly so that a profiler's launch list shows every kernel.
"""

from __future__ import annotations

import argparse
import dataclasses
import random

import torch

from _common import emit

from daser_b200.engine.runner import GpuModelRunner
from daser_b200.models.llama import PRESETS, LlamaWeights
from daser_b200.ops import gemm


def shard_config(cfg, tp: int):
    return dataclasses.replace(cfg, name=f"{cfg.name}/tp{tp}-shard", num_heads=cfg.num_heads // tp,
                               num_kv_heads=max(1, cfg.num_kv_heads // tp), intermediate=cfg.intermediate // tp,
                               vocab_size=cfg.vocab_size // tp)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--tp", default="1,2,4,8")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=3328)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--launches", action="store_true", help="one more, eager, step at the end (for a launch list)")
    args = ap.parse_args()
    base = PRESETS[args.model]
    bt = base.block_tokens
    ctx_tokens = -(-args.ctx // bt) * bt
    n_blocks = ctx_tokens // bt
    rng = random.Random(0)
    for tp in [int(t) for t in args.tp.split(",")]:
        cfg = shard_config(base, tp)
        w = LlamaWeights.random(cfg, "cuda", torch.bfloat16, seed=1)
        if w.inter_local % gemm.GATE_UP_BLOCK == 0:
            w.interleave_gate_up_(gemm.GATE_UP_BLOCK)
        runner = GpuModelRunner(cfg, w, n_blocks + 8, max(256, args.tokens), 8, max_blocks=max(512, n_blocks + 8))
        seq = [{"tokens": [rng.randrange(cfg.vocab_size) for _ in range(args.tokens)],
                "start_pos": ctx_tokens - args.tokens, "block_table": list(range(n_blocks))}]
        for _ in range(4):  # eager, capture, two replays
            runner.forward(runner.stage_inputs(seq))
        torch.cuda.synchronize()
        times = []
        for _ in range(args.iters):
            inp = runner.stage_inputs(seq)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.forward(inp)
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        runner.check_status()
        times.sort()
        weights_gb = sum(t.numel() * 2 for lw in w.layers for t in (lw.wqkv, lw.wo, lw.w_gate_up, lw.w_down)) / 1e9
        emit({"bench": "step_shapes", "model": cfg.name, "tp_shard": tp, "tokens": args.tokens, "ctx": ctx_tokens,
              "ms_median": times[len(times) // 2], "ms_best": times[0], "layer_weights_GB": weights_gb,
              "us_per_layer": times[len(times) // 2] * 1e3 / cfg.num_layers})
        if args.launches:
            runner.use_graphs = False
            runner.forward(runner.stage_inputs(seq))
            torch.cuda.synchronize()
        del runner, w
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
