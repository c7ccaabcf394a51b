"""The forms of the tensor-parallel reduction, side by side in one launch.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_tp_forms.py [--model llama3-70b] [--tokens 64] [--ctx 3328] [--iters 20]

One process per GPU builds its weight shard once, then times the model forward of a
``--tokens``-token step over a ``--ctx``-token context (the compute part of the RAG time to first
token; no store, no restore) with each arrangement in turn:

* ``twoshot``  GEMM epilogue reduce-scatter into the owner's slots + all-gather push gated on flags
* ``oneshot``  GEMM epilogue stores the partial into every rank's slot, each rank sums locally
* ``nvls``     (only when named in ``--forms``) the partial stays in the rank's own buffer, every
               rank reads the sum through the NVLink multicast mapping (``multimem.ld_reduce``)
* ``nccl``     the unfused baseline: same kernels, NCCL all-reduce of the row-parallel outputs

Every arrangement is warmed up until its CUDA graph is captured, then timed with CUDA events
around each replay; the figure printed is the median over iterations of the maximum over ranks.
The KV pool holds zeros except for the step's own tokens (random weights, synthetic tokens):
attention reads the same number of bytes whatever they contain, and every arrangement reads the
same ones.
"""

from __future__ import annotations

import argparse
import os
import random

import torch
import torch.distributed as dist

from _common import emit

from daser_b200.engine.runner import GpuModelRunner
from daser_b200.models.llama import PRESETS, LlamaWeights
from daser_b200.ops import gemm
from daser_b200.parallel.tp import TPContext


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-70b", choices=sorted(PRESETS))
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=3328)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--forms", default="twoshot,oneshot,nccl")
    args = ap.parse_args()
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tp = dist.get_world_size()
    cfg = PRESETS[args.model]
    bt = cfg.block_tokens
    ctx_tokens = -(-args.ctx // bt) * bt
    n_blocks = ctx_tokens // bt
    forms = [f for f in args.forms.split(",") if f]
    ctx = TPContext(cfg, dist.group.WORLD, max_tokens=max(256, args.tokens), multicast="nvls" in forms)
    weights = LlamaWeights.random(cfg, "cuda", torch.bfloat16, tp=tp, rank=rank, seed=1)
    if weights.inter_local % gemm.GATE_UP_BLOCK == 0:
        weights.interleave_gate_up_(gemm.GATE_UP_BLOCK)
    rng = random.Random(0)
    table = list(range(n_blocks))
    step_tokens = [rng.randrange(cfg.vocab_size) for _ in range(args.tokens)]
    results = {}
    for form in forms:
        ctx.impl = form
        runner = GpuModelRunner(cfg, weights, n_blocks + 8, max(256, args.tokens), 8, ctx,
                                max_blocks=max(512, n_blocks + 8))
        seq = [{"tokens": step_tokens, "start_pos": ctx_tokens - args.tokens, "block_table": table}]
        for _ in range(4):  # eager, capture, two replays
            runner.forward(runner.stage_inputs(seq))
        torch.cuda.synchronize()
        ctx.barrier()
        times = []
        for _ in range(args.iters):
            inp = runner.stage_inputs(seq)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ctx.barrier()
            s.record()
            runner.forward(inp)
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t.item()))
        runner.check_status()
        times.sort()
        results[form] = times[len(times) // 2]
        if rank == 0:
            emit({"bench": "tp_forward", "form": form, "tp": tp, "model": cfg.name, "tokens": args.tokens,
                  "ctx": ctx_tokens, "ms_median_max_over_ranks": results[form], "ms_best": times[0]})
        del runner
        torch.cuda.empty_cache()
    ctx.close()
    ctx.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
