"""fp8 paged decode attention micro-benchmark against the HBM-bandwidth roofline.

    python benchmarks/bench_decode_attn.py [--batch 64] [--min-ctx 4096] [--max-ctx 32768]

Batch 64, context lengths uniform in [4k, 32k], GQA 64 query / 8 KV heads, head_dim 128,
16-token pages; KV drawn N(0,1) then block-scale quantised (e4m3 + one fp32 scale per 16
elements), queries bf16 N(0,1).  Algorithmic bytes = sum(ctx) * 2 (K,V) * 8 heads * 128 * 1.25
plus q and o; the fraction is of the measured copy bandwidth.  The reference serves decode
attention from stock vLLM over a bf16 cache (2 bytes per element).
"""

from __future__ import annotations

import argparse
import random

import torch

from _common import emit, peaks, time_cuda

from daser_b200.ops import attention, kv_ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--min-ctx", type=int, default=4096)
    ap.add_argument("--max-ctx", type=int, default=32768)
    ap.add_argument("--hq", type=int, default=64)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--splits", default="")
    args = ap.parse_args()
    rng = random.Random(args.seed)
    D, B = 128, 16
    ctx = [rng.randint(args.min_ctx, args.max_ctx) for _ in range(args.batch)]
    blocks = [-(-c // B) for c in ctx]
    n_blocks = sum(blocks)
    dev = "cuda"
    # fill the pool on the device: N(0,1) -> fp8b16 with the library's own codec kernel
    payload = torch.empty(1, n_blocks, 2, args.hkv, B, D, dtype=torch.uint8, device=dev)
    scales = torch.empty(1, n_blocks, 2, args.hkv, B, D // 16, dtype=torch.float32, device=dev)
    step = 2048
    for i in range(0, n_blocks, step):
        x = torch.randn(min(step, n_blocks - i), 2, args.hkv, B, D, device=dev).to(torch.bfloat16)
        q8, sc = kv_ops.quantize_fp8b16(x)
        payload[0, i : i + x.shape[0]] = q8
        scales[0, i : i + x.shape[0]] = sc
    pool = kv_ops.PagedKVPool.from_tensors([payload], [scales], "LNKHTD")
    perm = torch.randperm(n_blocks).tolist()
    tables = torch.zeros(args.batch, max(blocks), dtype=torch.int32)
    used = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = torch.tensor(perm[used : used + nb], dtype=torch.int32)
        used += nb
    tables = tables.to(dev)
    q = torch.randn(args.batch, args.hq, D, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    q_start = torch.arange(args.batch + 1, dtype=torch.int32, device=dev)
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=dev)
    ws = attention.AttentionWorkspace(dev)
    hbm, _, kind = peaks()
    kv_bytes = sum(ctx) * 2 * args.hkv * D * 1.25
    total_bytes = kv_bytes + 2 * q.numel() * 2
    plans = [None]
    if args.splits:
        plans = [tuple(int(v) for v in p.split("x")) for p in args.splits.split(",")]
    for plan in plans:
        kw = {}
        if plan is not None:
            kw = dict(nsplit=plan[0], split_tokens=plan[1])
        else:
            ns, st = attention.plan_splits(args.batch, args.hkv, 1, args.hq // args.hkv, max(ctx), B)
            kw = dict(nsplit=ns, split_tokens=st)
        fn = lambda: attention.paged_attention(q, out, pool, 0, tables, q_start, ctx_t, 1, max(ctx), args.hkv,
                                               D**-0.5, ws, **kw)
        med, best = time_cuda(fn, iters=10, warmup=3, flush=True)
        emit({"kernel": "paged_attn_fp8(decode)", "batch": args.batch, "sum_ctx": sum(ctx), "max_ctx": max(ctx),
              "nsplit": kw["nsplit"], "split_tokens": kw["split_tokens"], "ms": med, "best_ms": best,
              "GBps": total_bytes / med / 1e6, f"frac_of_{kind}_hbm": total_bytes / med / 1e6 / hbm,
              "kv_GB": kv_bytes / 1e9, "l2": "KV pool (GBs) larger than L2 and flushed between launches"})


if __name__ == "__main__":
    main()
