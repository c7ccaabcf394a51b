"""Open-loop RAG serving benchmark: Poisson arrivals, continuous batching, TTFT percentiles.

    python benchmarks/bench_rag_serving.py [--model llama3-8b] [--rate 4] [--requests 64] [--k 5]

The workload of the single-GPU serving configuration: a pool of lognormal-length chunks
(median 300 tokens, sigma 0.6, clipped to 64..1024), each request = a 64-token system prefix +
k chunks drawn Zipf(s = 1.1) + a 64-token query, 128 output tokens, Poisson arrivals at ``rate``
requests per second.  KV is stored block-scaled fp8 and restored through the tiers.  The engine
admits a waiting request with one TTFT step and otherwise decodes all running sequences as a
batch.  TTFT is measured from the request's arrival time to its first token (wall clock,
including queueing).  The pool is scaled down from 20k chunks so that filling it fits the run;
its size is printed.
"""

from __future__ import annotations

import argparse
import asyncio
import os
import random
import sys
import tempfile
import threading
import time

import torch

from _common import emit, percentile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bench import make_traffic  # noqa: E402

from daser_b200.config import DaserConfig  # noqa: E402
from daser_b200.engine.rag_gpu import GpuRagEngine, RagRequest  # noqa: E402
from daser_b200.models.llama import PRESETS  # noqa: E402
from daser_b200.server.__main__ import ControlPlane  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--k", type=int, default=5)
    ap.add_argument("--pool", type=int, default=128)
    ap.add_argument("--output-tokens", type=int, default=128)
    args = ap.parse_args()
    cfg = PRESETS[args.model]
    bt = cfg.block_tokens
    prefix, pool, reqs = make_traffic(cfg, args.pool, args.k, args.requests)
    slot = cfg.num_layers * 2 * bt * cfg.num_kv_heads * cfg.head_dim * 5 // 4
    pool_slots = sum(len(c) // bt for c in pool) + len(prefix) // bt
    tmp = tempfile.mkdtemp(prefix="daser_serve_")
    dcfg = DaserConfig(store_path=f"{tmp}/daser.store", index_path="", total_slots=pool_slots + 64, slot_size=slot,
                       ipc_socket_path=f"{tmp}/d.sock", block_tokens=bt, codec="fp8b16", log_level="WARNING")
    os.environ.setdefault("DASER_LOG_LEVEL", "WARNING")
    plane = ControlPlane(dcfg)
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def serve():
        asyncio.set_event_loop(loop)
        loop.run_until_complete(plane.start())
        ready.set()
        loop.run_forever()

    threading.Thread(target=serve, daemon=True).start()
    ready.wait(30)
    from daser_b200.io.engine import preallocate

    preallocate(dcfg.store_path, dcfg.total_slots * slot)
    per_req_blocks = -(-(args.k * 1024 + 128 + args.output_tokens) // bt)
    eng = GpuRagEngine(cfg, dcfg.ipc_socket_path, dcfg.store_path, num_blocks=per_req_blocks * 24, max_tokens=256,
                       max_seqs=32, hbm_slots=pool_slots // 2, host_slots=pool_slots, staging_slots=per_req_blocks)
    t0 = time.time()
    for c in [prefix] + pool:
        eng.store_chunk(c)
    fill_s = time.time() - t0
    eng.warm_up(token_counts=(64,), context_lens=(2048, 4096, 8192))
    for n in (1, 2, 4, 8, 16):  # decode batch shapes
        tables = [eng.blocks.alloc(130) for _ in range(n)]
        for _ in range(3):
            eng.runner.forward(eng.runner.stage_inputs(
                [{"tokens": [1], "start_pos": 2000, "block_table": t} for t in tables]))
        for t in tables:
            eng.blocks.free(t)
    torch.cuda.synchronize()

    rng = random.Random(1)
    arrivals, t = [], 0.0
    for _ in reqs:
        t += rng.expovariate(args.rate)
        arrivals.append(t)
    pending = list(zip(arrivals, reqs))
    live: list[tuple[float, RagRequest]] = []
    done: list[tuple[float, RagRequest, float]] = []
    first_seen: dict[str, float] = {}
    start = time.perf_counter()
    while pending or eng.has_work():
        now = time.perf_counter() - start
        while pending and pending[0][0] <= now:
            at, (chunks, query) = pending.pop(0)
            r = eng.submit(RagRequest([list(c) for c in chunks], list(query), args.output_tokens))
            live.append((at, r))
        if eng.has_work():
            eng.step()
            now = time.perf_counter() - start
            for at, r in live:
                if r.generated and r.req_id not in first_seen:
                    first_seen[r.req_id] = now - at
            for item in [x for x in live if x[1].done]:
                live.remove(item)
                done.append((item[0], item[1], now))
        elif pending:
            time.sleep(max(0.0, min(0.002, pending[0][0] - now)))
    wall = time.perf_counter() - start
    ttft = [v * 1e3 for v in first_seen.values()]
    gen = sum(len(r.generated) for _, r, _ in done)
    emit({"bench": "rag_serving", "model": cfg.name, "rate_req_s": args.rate, "requests": len(done),
          "chunks_per_request": args.k, "chunk_pool": args.pool, "output_tokens": args.output_tokens,
          "ttft_p50_ms": percentile(ttft, 50), "ttft_p99_ms": percentile(ttft, 99),
          "ttft_step_p50_ms": percentile([r.ttft_ms for _, r, _ in done], 50),
          "restored_chunks_per_request": sum(r.restored_chunks for _, r, _ in done) / max(len(done), 1),
          "output_tok_s": gen / wall, "wall_s": wall, "fill_s": fill_s,
          "io_backend": eng.worker.transfer.backend.name, "kv_codec": "fp8b16"})
    eng.close()
    asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
    loop.call_soon_threadsafe(loop.stop)


if __name__ == "__main__":
    main()
