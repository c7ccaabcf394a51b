"""This package's connector inside a stock ``vllm.LLM``: cold pass, then the timed warm pass.

    python benchmarks/bench_vllm_connector.py [--model llama3-70b] [--steps 8] [--warmup 2]
                                              [--codec fp8b16] [--host-slots -1] [--hbm-slots 0]

The same protocol, traffic and engine settings as the reference arm of the headline benchmark
(``baseline/reference_arm.py``; the reference's own end-to-end benchmark is
``benchmarks/bench_e2e_daser_vs_lmcache.py:404-466``): every request is served once cold (prefill,
fused save kernel, store file, commit) and then again with the identical prompt, which is the
only kind of hit a stock vLLM scheduler can be offered; the warm pass is timed, one request at a
time, wall clock around ``LLM.generate(max_tokens=1)``.  What differs from that arm is the
connector and the control plane only, so the two warm numbers compare connector against
connector under one engine.

``--host-slots -1`` sizes the pinned host tier for the run's working set (the reference's warm
pass reads its file through the page cache, which is host memory too); ``--host-slots 0`` leaves
the store file (O_DIRECT, io_uring) as the only source.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import shutil
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

BLOCK_TOKENS = 16


class Plane:
    """The control plane on a thread of this process."""

    def __init__(self, tmpdir: str, total_slots: int, slot_size: int) -> None:
        from daser_b200.config import DaserConfig
        from daser_b200.server.__main__ import ControlPlane

        self.cfg = DaserConfig(store_path=os.path.join(tmpdir, "daser.store"),
                               index_path=os.path.join(tmpdir, "daser.index"), total_slots=total_slots,
                               slot_size=slot_size, ipc_socket_path=os.path.join(tmpdir, "d.sock"),
                               block_tokens=BLOCK_TOKENS)
        self.plane = ControlPlane(self.cfg)
        self.loop = asyncio.new_event_loop()
        self._ready = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        asyncio.set_event_loop(self.loop)
        self.loop.run_until_complete(self.plane.start())
        self._ready.set()
        self.loop.run_forever()

    def start(self) -> "Plane":
        self.thread.start()
        if not self._ready.wait(20):
            raise RuntimeError("control plane did not start")
        return self

    def stop(self) -> None:
        asyncio.run_coroutine_threadsafe(self.plane.stop(save=False), self.loop).result(10)
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.thread.join(10)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--pool", type=int, default=128)
    ap.add_argument("--k", type=int, default=8)
    ap.add_argument("--codec", default="fp8b16", choices=("raw", "fp8b16"))
    ap.add_argument("--host-slots", type=int, default=-1)
    ap.add_argument("--hbm-slots", type=int, default=0)
    ap.add_argument("--backend", default="FLASH_ATTN")
    ap.add_argument("--gpu-util", type=float, default=0.92)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--write-behind", type=int, default=1, help="0: wait for the file write inside wait_for_save")
    args = ap.parse_args()

    import vllm_common as vc
    from traffic import MODEL_SHAPES, make_traffic, percentile

    shape = MODEL_SHAPES[args.model]
    tp = args.gpus
    n_req = args.steps + args.warmup
    _, _, reqs = make_traffic(shape["vocab_size"], BLOCK_TOKENS, args.pool, args.k, n_req)
    prompts = [[t for c in chunks for t in c] + query[:-1] for chunks, query, _ in reqs]
    max_model_len = -(-(max(map(len, prompts)) + 16) // 1024) * 1024
    raw_slot = vc.slot_size_bf16(args.model, BLOCK_TOKENS, tp)
    slot = raw_slot if args.codec == "raw" else raw_slot * 5 // 8  # e4m3 + one fp32 scale per 16 elements
    need_slots = sum(-(-len(p) // BLOCK_TOKENS) for p in prompts) + 64
    host_slots = need_slots if args.host_slots < 0 else args.host_slots
    tmpdir = tempfile.mkdtemp(prefix="daser_vllm_")
    if need_slots * slot > shutil.disk_usage(tmpdir).free * 0.9:
        raise RuntimeError(f"store of {need_slots * slot >> 20} MiB does not fit {tmpdir}")
    plane = Plane(tmpdir, need_slots, slot).start()
    model_dir = vc.write_hf_config(args.model, os.path.join(tmpdir, "model"))
    ktc = {
        "kv_connector": "DaserConnector",
        "kv_connector_module_path": "daser_b200.connector.daser_connector",
        "kv_role": "kv_both",
        "kv_connector_extra_config": {"socket_path": plane.cfg.ipc_socket_path, "store_path": plane.cfg.store_path,
                                      "slot_size": slot, "block_tokens": BLOCK_TOKENS, "model_id": args.model,
                                      "codec": args.codec, "hbm_slots": args.hbm_slots, "host_slots": host_slots,
                                      # one prompt's blocks fit the pinned arena (longer ones would go in pieces)
                                      "staging_slots": (2 if args.write_behind else 1)
                                      * max(-(-len(p) // BLOCK_TOKENS) for p in prompts),
                                      "write_behind": bool(args.write_behind)},
    }
    env = vc.clean_env([ROOT, os.path.join(ROOT, "baseline")])  # the engine's children inherit it
    for k in [k for k in os.environ if k not in env]:
        del os.environ[k]
    os.environ.update(env)
    t0 = time.time()
    llm = vc.build_llm(model_dir, tp, ktc, max_model_len, gpu_memory_utilization=args.gpu_util,
                       attention_backend=args.backend, enforce_eager=args.eager)
    init_s = time.time() - t0
    try:
        vc.first_token_ms(llm, [5] * 40)
        t0 = time.time()
        cold = [vc.first_token_ms(llm, p) for p in prompts]
        cold_s = time.time() - t0
        for p in prompts[: args.warmup]:
            vc.first_token_ms(llm, p)
        sampler = vc.ClockSampler(0)
        sampler.start()
        warm = [vc.first_token_ms(llm, p) for p in prompts[args.warmup:]]
        clocks = sampler.stop()
    finally:
        vc.destroy_llm(llm)
        plane.stop()
    warm_ms = [m for m, _ in warm]
    cold_ms = [m for m, _ in cold[args.warmup:]]
    timed = prompts[args.warmup:]
    restored = sum((len(p) // BLOCK_TOKENS) * slot * tp for p in timed)
    print(json.dumps({
        "bench": "vllm_connector", "model": args.model, "n_gpus": tp, "codec": args.codec,
        "attention_backend": args.backend, "host_slots": host_slots, "hbm_slots": args.hbm_slots, "write_behind": bool(args.write_behind),
        "warm_ttft_ms": {"p50": round(percentile(warm_ms, 50), 3), "p99": round(percentile(warm_ms, 99), 3)},
        "cold_ttft_ms": {"p50": round(percentile(cold_ms, 50), 3), "p99": round(percentile(cold_ms, 99), 3)},
        "kv_restore_gbs": round(restored / (sum(warm_ms) / 1e3) / 1e9, 3),
        "prompt_tokens_mean": int(sum(map(len, timed)) / len(timed)),
        "cold_vs_warm_first_token_mismatches": f"{sum(1 for (_, a), (_, b) in zip(cold[args.warmup:], warm) if a != b)}/{len(warm)}",
        "slot_size": slot, "store_MB": need_slots * slot >> 20, "init_s": round(init_s, 1),
        "cold_pass_s": round(cold_s, 1), "enforce_eager": bool(args.eager), "clocks": clocks,
        "timing": "wall clock around LLM.generate(max_tokens=1), one request at a time",
    }), flush=True)
    shutil.rmtree(tmpdir, ignore_errors=True)


if __name__ == "__main__":
    main()
