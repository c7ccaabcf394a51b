"""End-to-end cold / warm benchmark through the native engine.

    python benchmarks/bench_e2e.py [--model llama3-8b] [--prompts 200] [--mean-tokens 303]

Counterpart of the reference's ``benchmarks/bench_e2e_daser_vs_lmcache.py`` (DaseR side):
the same engine serves N prompts twice with ``max_tokens = 1`` — a cold pass in which every
prompt misses, is computed and stored, then a warm pass in which the block-aligned part of
every prompt is restored from the store and only the tail is computed.  Reports prompt
tokens/s of both passes, the warm/cold speed-up and how many first tokens differ between the
passes.  The reference's published run (H800, Qwen3-8B, 200 IMDB prompts of ~303 tokens) gave
8 940 tok/s cold and 28 772 tok/s warm; prompts here are synthetic token ids of the same
length distribution because no dataset is available offline.  ``--model qwen3-8b`` runs the
reference's own architecture (random-init weights); the default stays the Llama-3-8B shape that
the recorded figures were taken with.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import tempfile
import threading
import time

import torch

from _common import emit

from daser_b200.config import DaserConfig
from daser_b200.engine.rag_gpu import GpuRagEngine
from daser_b200.models.llama import PRESETS
from daser_b200.server.__main__ import ControlPlane


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--prompts", type=int, default=200)
    ap.add_argument("--mean-tokens", type=int, default=303)
    ap.add_argument("--hbm-slots", type=int, default=0, help="0 = warm pass reads the store file / host tier")
    ap.add_argument("--host-slots", type=int, default=0)
    ap.add_argument("--write-behind", type=int, default=1, help="0: a store waits for its file write")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    cfg = PRESETS[args.model]
    bt = cfg.block_tokens
    rng = random.Random(0)
    prompts = []
    for _ in range(args.prompts):
        n = max(2 * bt + 1, int(rng.gauss(args.mean_tokens, args.mean_tokens * 0.45)))
        prompts.append([rng.randrange(1, cfg.vocab_size) for _ in range(n)])
    total_tokens = sum(len(p) for p in prompts)
    total_blocks = sum(len(p) // bt for p in prompts)
    slot = cfg.num_layers * 2 * bt * cfg.num_kv_heads * cfg.head_dim * 5 // 4
    tmp = tempfile.mkdtemp(prefix="daser_e2e_")
    dcfg = DaserConfig(store_path=f"{tmp}/daser.store", index_path="", total_slots=total_blocks + 64, slot_size=slot,
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
    eng = GpuRagEngine(cfg, dcfg.ipc_socket_path, dcfg.store_path, num_blocks=512, max_tokens=512, max_seqs=8,
                       hbm_slots=args.hbm_slots, host_slots=args.host_slots, staging_slots=256,
                       write_behind=bool(args.write_behind))

    def run_pass(store):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        firsts, restored = [], 0
        sums: dict = {}
        for p in prompts:
            aligned = ((len(p) - 1) // bt) * bt  # at least one token is always computed
            req = eng.generate([p[:aligned]], p[aligned:], max_new_tokens=1, store_misses=store)
            firsts.append(req.generated[0])
            restored += req.restored_chunks
            for k, v in req.timings.items():
                sums[k] = sums.get(k, 0.0) + v
            sums["ttft_ms"] = sums.get("ttft_ms", 0.0) + req.ttft_ms
        eng.worker.flush_stores()  # the pass ends when its last chunk is on the drive and committed
        torch.cuda.synchronize()
        mean = {k: round(v / len(prompts), 3) for k, v in sums.items() if k.endswith("_ms")}
        return time.perf_counter() - t0, firsts, restored, mean

    # warm the kernels (not the cache) on a throw-away prompt
    eng.generate([[1] * (4 * bt)], [2, 3, 4], 1)
    cold_s, cold_tok, cold_hits, cold_mean = run_pass(store=True)
    warm_s, warm_tok, warm_hits, warm_mean = run_pass(store=False)
    row = {
        "bench": "e2e_cold_warm", "model": cfg.name, "prompts": args.prompts, "prompt_tokens": total_tokens,
        "kv_blocks": total_blocks, "cold_s": cold_s, "warm_s": warm_s, "cold_tok_s": total_tokens / cold_s,
        "warm_tok_s": total_tokens / warm_s, "warm_over_cold": cold_s / warm_s, "cold_hits": cold_hits,
        "warm_hits": warm_hits, "first_token_mismatches": sum(a != b for a, b in zip(cold_tok, warm_tok)),
        "io_backend": eng.worker.transfer.backend.name, "kv_codec": "fp8b16", "write_behind": bool(args.write_behind),
        "cold_mean_ms_per_prompt": cold_mean, "warm_mean_ms_per_prompt": warm_mean,
        "reference_published": {"cold_tok_s": 8940, "warm_tok_s": 28772, "hardware": "1x H800, Qwen3-8B"},
    }
    emit(row)
    if args.json:
        json.dump(row, open(args.json, "w"), indent=1)
    eng.close()
    asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
    loop.call_soon_threadsafe(loop.stop)


if __name__ == "__main__":
    main()
