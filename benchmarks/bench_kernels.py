"""Device-timed micro-benchmarks of the hand-written kernels against their rooflines.

    python benchmarks/bench_kernels.py [--quick] [--only restore,gemm,...] [--json out.json]

Each kernel is timed with CUDA events after 3 warm-up launches; between timed launches a
buffer larger than L2 is rewritten so no input is served from cache.  Fractions are
"of measured": the denominators come from ``MEASURED_PEAKS.json`` next to the repository
root when present (copy bandwidth and cuBLAS bf16 throughput measured on this pool),
else the fallback 6650 GB/s and 1590 TFLOP/s.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from daser_b200.kv.layout import KVGeometry  # noqa: E402
from daser_b200.ops import elementwise as ew  # noqa: E402
from daser_b200.ops import gemm, kv_ops  # noqa: E402
from daser_b200.position import inv_freq_table  # noqa: E402


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def time_ms(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def bench_codec(out, quick):
    hbm, _, kind = peaks()
    n = (256 if quick else 1024) * 1024 * 1024 // 2
    x = (torch.randn(n // 128, 128, device="cuda") * 0.5).to(torch.bfloat16)
    med, best = time_ms(lambda: kv_ops.quantize_fp8b16(x))
    bytes_ = n * 2 + n + n // 4
    out.append({"kernel": "quant_fp8b16", "elems": n, "ms": med, "GBps": bytes_ / med / 1e6,
                f"frac_of_{kind}_hbm": bytes_ / med / 1e6 / hbm})


def bench_restore(out, quick):
    hbm, _, kind = peaks()
    # Llama-3-70B geometry, one 2k-token context (128 slots) per launch
    for img_codec, pool_fp8, tp in [("fp8b16", True, 1), ("fp8b16", False, 1), ("raw", False, 1), ("fp8b16", True, 8)]:
        geo = KVGeometry(80, 8, 128, 16, 2, img_codec)
        n_slots = 32 if quick else 128
        n_blocks = n_slots + 8
        staging = torch.randint(0, 120, (n_slots * geo.slot_size,), dtype=torch.uint8, device="cuda")
        hn = 8 // tp
        if pool_fp8:
            payloads = [torch.zeros(80, n_blocks, 2, hn, 16, 128, dtype=torch.uint8, device="cuda") for _ in range(tp)]
            scales = [torch.zeros(80, n_blocks, 2, hn, 16, 8, dtype=torch.float32, device="cuda") for _ in range(tp)]
        else:
            payloads = [torch.zeros(80, n_blocks, 2, hn, 16, 128, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
            scales = None
        pool = kv_ops.PagedKVPool.from_tensors(payloads, scales, "LNKHTD")
        work = kv_ops.KVWorkList(
            torch.tensor([staging.data_ptr() + i * geo.slot_size for i in range(n_slots)], dtype=torch.int64, device="cuda"),
            torch.randperm(n_blocks, device="cuda")[:n_slots].to(torch.int32),
            torch.full((n_slots,), 777, dtype=torch.int32, device="cuda"),
        )
        cos_sin = kv_ops.rope_table(8192, inv_freq_table(128, 500000.0), "cuda")
        status = torch.zeros(2, dtype=torch.int32, device="cuda")
        med, best = time_ms(lambda: kv_ops.kv_restore(work, geo, pool, cos_sin, status))
        assert status.tolist() == [0, 0]
        elems = n_slots * 80 * geo.elems_per_layer
        rd = n_slots * geo.slot_size
        wr = elems * (1.25 if pool_fp8 else 2)
        out.append({"kernel": "kv_restore", "image": img_codec, "pool": "fp8b16" if pool_fp8 else "bf16",
                    "tp_emulated": tp, "slots": n_slots, "ms": med, "image_GBps": rd / med / 1e6,
                    "total_GBps": (rd + wr) / med / 1e6, f"frac_of_{kind}_hbm": (rd + wr) / med / 1e6 / hbm})
        med, best = time_ms(lambda: kv_ops.kv_save(work, geo, pool, 0, status))
        frac_heads = 1.0 / tp
        out.append({"kernel": "kv_save(rank0)", "image": img_codec, "pool": "fp8b16" if pool_fp8 else "bf16",
                    "tp_emulated": tp, "slots": n_slots, "ms": med,
                    "total_GBps": (rd + wr) * frac_heads / med / 1e6,
                    f"frac_of_{kind}_hbm": (rd + wr) * frac_heads / med / 1e6 / hbm})
        del payloads, scales, staging


def bench_gemm(out, quick):
    hbm, tflops, kind = peaks()
    shapes = [
        # (M, N, K, label)  Llama-3-70B layers, TP=1 and TP=8 shards, TTFT tail of 64 tokens
        (64, 10240, 8192, "qkv tp1 M64"), (64, 8192, 8192, "o tp1 M64"),
        (64, 57344, 8192, "gate_up tp1 M64"), (64, 8192, 28672, "down tp1 M64"),
        (64, 1280, 8192, "qkv tp8 M64"), (64, 8192, 1024, "o tp8 M64"),
        (64, 7168, 8192, "gate_up tp8 M64"), (64, 8192, 3584, "down tp8 M64"),
        (2048, 10240, 8192, "qkv tp1 M2048"), (2048, 8192, 28672, "down tp1 M2048"),
        (8192, 8192, 8192, "square 8192"),
    ]
    if quick:
        shapes = shapes[4:9]
    for M, N, K, label in shapes:
        x = (torch.randn(M, K, device="cuda") * 0.1).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (M * K + N * K + M * N)
        row = {"kernel": "gemm_tcgen05", "shape": [M, N, K], "label": label}
        bn, ks = gemm.plan_tiles(M, N, K, allow_split=True)
        if ks > 1:
            acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
            fn = lambda: gemm.linear(x, w, acc=acc, block_n=bn, k_splits=ks)
        else:
            o = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            fn = lambda: gemm.linear(x, w, out=o, block_n=bn, k_splits=1)
        med, best = time_ms(fn)
        row.update({"block_n": bn, "k_splits": ks, "ms": med, "TFLOPs": flops / med / 1e9,
                    "GBps": bytes_ / med / 1e6,
                    f"frac_of_{kind}": max(flops / med / 1e9 / tflops, bytes_ / med / 1e6 / hbm)})
        med_t, _ = time_ms(lambda: torch.matmul(x, w.t()))
        row.update({"torch_ms": med_t, "vs_torch": med_t / med})
        out.append(row)
        del x, w


def bench_norm(out, quick):
    hbm, _, kind = peaks()
    T, H = (4096 if quick else 32768), 8192
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    o = torch.empty_like(x)
    med, _ = time_ms(lambda: ew.add_rmsnorm(x, w, residual=res, out=o))
    bytes_ = T * H * 2 * 4
    out.append({"kernel": "add_rmsnorm", "shape": [T, H], "ms": med, "GBps": bytes_ / med / 1e6,
                f"frac_of_{kind}_hbm": bytes_ / med / 1e6 / hbm})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default="codec,restore,gemm,norm")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rows = []
    table = {"codec": bench_codec, "restore": bench_restore, "gemm": bench_gemm, "norm": bench_norm}
    for name in args.only.split(","):
        try:
            table[name](rows, args.quick)
        except Exception as exc:  # keep going: one failing kernel must not hide the others
            rows.append({"kernel": name, "error": repr(exc)})
        for r in rows:
            if not r.get("_printed"):
                print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}), flush=True)
                r["_printed"] = True
    if args.json:
        for r in rows:
            r.pop("_printed", None)
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
