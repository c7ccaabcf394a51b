"""Chunked-prefill attention micro-benchmark: a short query block over a long restored context.

    python benchmarks/bench_prefill_attn.py [--q 64] [--ctx 3328] [--hq 64] [--hkv 8]

This is the attention call of the RAG time-to-first-token step: the chunk KV was restored into
the fp8 pool and only the query tokens are computed.  Both kernels are timed on the same
inputs: the tcgen05/TMEM one and the mma.sync one it replaces, each with the split plan the
library picks for it, L2 flushed before every timed launch.  The error column is against fp32
attention over the dequantised cache.  The reference runs this step through stock vLLM's
FlashAttention kernel over a bf16 cache.
"""

from __future__ import annotations

import argparse

import torch

from _common import emit, time_cuda

from daser_b200.kv import codec
from daser_b200.ops import attention, kv_ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--q", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=3328)
    ap.add_argument("--hq", type=int, default=64)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--check", type=int, default=1)
    ap.add_argument("--plans", default="", help="extra split plans for the tcgen05 kernel, e.g. 26x128,9x384")
    args = ap.parse_args()
    D, B, dev = 128, 16, "cuda"
    nb = -(-args.ctx // B)
    torch.manual_seed(0)
    x = torch.randn(1, nb, 2, args.hkv, B, D, device=dev).to(torch.bfloat16)
    payload, scales = kv_ops.quantize_fp8b16(x)
    pool = kv_ops.PagedKVPool.from_tensors([payload], [scales], "LNKHTD")
    tables = torch.randperm(nb, device=dev).to(torch.int32)[None].contiguous()
    q = torch.randn(args.q, args.hq, D, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    q_start = torch.tensor([0, args.q], dtype=torch.int32, device=dev)
    ctx_t = torch.tensor([args.ctx], dtype=torch.int32, device=dev)
    ws = attention.AttentionWorkspace(dev)
    ref = None
    if args.check:
        deq = codec.dequantize_fp8b16(payload.cpu(), scales.cpu())[0, tables[0].cpu().long()]  # [nb, 2, H, B, D]
        kv = deq.permute(1, 0, 3, 2, 4).reshape(2, nb * B, args.hkv, D)[:, : args.ctx]
        g = args.hq // args.hkv
        k, v = kv[0].repeat_interleave(g, 1), kv[1].repeat_interleave(g, 1)
        sc = torch.einsum("thd,shd->hts", q.float().cpu(), k) * D**-0.5
        lim = (args.ctx - args.q + torch.arange(args.q))[:, None]
        sc = sc.masked_fill((torch.arange(args.ctx)[None, :] > lim)[None], float("-inf"))
        ref = torch.einsum("hts,shd->thd", sc.softmax(-1), v)
    flops = 4.0 * args.q * args.hq * args.ctx * D
    arms = [("tcgen05", True, None), ("mma.sync", False, None)]
    arms += [("tcgen05", True, tuple(int(v) for v in pl.split("x"))) for pl in args.plans.split(",") if pl]
    for name, tc, plan in arms:
        attention.set_tensor_core_prefill(tc)
        ns, st = plan or attention.plan_splits(1, args.hkv, args.q, args.hq // args.hkv, args.ctx, B)
        fn = lambda: attention.paged_attention(q, out, pool, 0, tables, q_start, ctx_t, args.q, args.ctx, args.hkv,
                                               D**-0.5, ws, nsplit=ns, split_tokens=st)
        med, best = time_cuda(fn, iters=20, warmup=3, flush=True)
        err = (out.float().cpu() - ref).abs().max().item() if ref is not None else None
        emit({"kernel": f"paged_attn_fp8(prefill, {name})", "q": args.q, "ctx": args.ctx, "hq": args.hq,
              "hkv": args.hkv, "nsplit": ns, "split_tokens": st, "us": med * 1e3, "best_us": best * 1e3,
              "TFLOPs": flops / med / 1e9, "max_abs_err": err, "tc_status": attention.tc_status()})
    attention.set_tensor_core_prefill(True)


if __name__ == "__main__":
    main()
