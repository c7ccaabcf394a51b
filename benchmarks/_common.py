"""Shared helpers of the benchmark scripts: peaks, device timing, percentiles."""

from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    """(HBM GB/s, bf16 TFLOP/s, "measured" | "fallback") — measured on this pool when the file exists."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def percentile(vals, q):
    v = sorted(vals)
    if not v:
        return 0.0
    return v[max(0, min(len(v) - 1, int(round(q / 100.0 * (len(v) - 1)))))]


_flush = None


def flush_l2():
    """Rewrite a buffer larger than L2 (126 MB) so the next kernel reads from HBM."""
    import torch

    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def time_cuda(fn, iters=10, warmup=3, flush=True):
    """(median ms, best ms) of ``fn`` timed with CUDA events on the current stream."""
    import torch

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


def emit(row: dict) -> None:
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
