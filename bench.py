"""Headline benchmark: RAG time-to-first-token and KV-restore rate, Llama-3-70B, TP = #GPUs.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the reference arm

A *step* is one RAG request served up to its first token through the engine's public call
(``GpuRagEngine.generate``): the control plane is asked for the request's chunks, the cached
chunks are read from the store (NVMe file or HBM tier) and restored at their new offsets by
the fused dequantise + RoPE-re-rotate + scatter kernel, the query is prefilled over the
restored context with the tcgen05 GEMMs and the fp8 paged attention, and the first token is
sampled and read back.

Traffic (synthetic, random-init weights): a 64-token system prefix + k chunks drawn
Zipf(s = 1.1) from a pool of lognormal-length chunks (median 300 tokens, sigma 0.6, clipped
to 64..1024, padded to whole 16-token blocks) + a 64-token query.  The pool is smaller than
the 20k chunks of the full workload so that filling it (real prefills through the save
kernel) fits the benchmark's time and the box's disk; its size is printed in ``config``.

Timing: W untimed warm-up steps, then exactly K timed steps between a barrier +
``torch.cuda.synchronize()`` on both sides.  ``value`` is the p50 over the K steps of the
device-timed TTFT (CUDA events on the launching stream, max over ranks); ``e2e.value`` is the
p50 wall-clock TTFT of the same steps including the pinned-host -> device copy of each
step's inputs and the device -> host read of the sampled token.  Weights (tens of GB per
GPU) are far larger than L2, so no input of a step is served from cache.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

from traffic import make_traffic, percentile  # noqa: E402
from vllm_common import ClockSampler  # noqa: E402

METRIC = "rag_ttft_p50_ms (Llama-3-70B, TP=#GPUs, chunk-KV restore from fp8 store)"


def reference_arm(args) -> None:
    """Runs ``baseline/reference_arm.py`` (the unmodified reference inside the stock ``vllm.LLM``)
    in a process of its own and relays its JSON line.

    vLLM starts and manages its own tensor-parallel workers, so under a multi-rank launcher only
    rank 0 acts, with the launcher's variables removed from the child's environment; the other
    ranks exit at once.  The child imports nothing of this framework: its ``PYTHONPATH`` holds
    the reference install and the kvikio / cupy stand-ins only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    base = os.path.join(ROOT, "baseline")
    sys.path.insert(0, base)
    out = None
    if not os.path.isdir(os.path.join(base, "_ref", "daser")):
        out = {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target of the reference)"}
    else:
        import vllm_common as vc

        env = vc.clean_env([os.path.join(base, "_ref"), os.path.join(base, "shims")])
        cmd = [sys.executable, os.path.join(base, "reference_arm.py"), "--gpus", str(args.gpus), "--steps",
               str(args.steps), "--warmup", str(max(args.warmup, 3)), "--model", args.model, "--pool", str(args.pool),
               "--k", str(args.k)]
        if args.store_dir:
            cmd += ["--store-dir", args.store_dir]
        if os.environ.get("DASER_REF_EAGER") == "1":
            cmd.append("--eager")
        # a session of its own: on a time-out the whole group goes (vLLM's engine and worker processes too)
        proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=None, text=True, start_new_session=True)
        try:
            stdout, _ = proc.communicate(timeout=float(os.environ.get("DASER_REF_TIMEOUT", "1500")))
            for line in stdout.splitlines():
                if line.startswith("REFERENCE_RESULT "):
                    out = json.loads(line[len("REFERENCE_RESULT "):])
            if out is None:
                out = {"impl": "reference", "unavailable": f"reference process ended with code {proc.returncode} and no result"}
        except subprocess.TimeoutExpired:
            import signal

            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait()
            out = {"impl": "reference", "unavailable": "reference process did not finish within its time limit"}
    print(json.dumps(out))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--pool", type=int, default=64, help="chunks in the synthetic pool")
    ap.add_argument("--tp-impl", choices=("fused", "twoshot", "oneshot", "nvls", "nccl"), default="fused",
                    help="fused: GEMM-epilogue reduction over peer memory (one-shot all-reduce for few tokens at "
                         "tp <= 2, reduce-scatter + gated all-gather otherwise); twoshot / oneshot: force one form; "
                         "nvls: partials stay local, each rank reads the sum through the NVLink multicast mapping; "
                         "nccl: the unfused baseline (same kernels, NCCL all-reduce)")
    ap.add_argument("--k", type=int, default=8, help="chunks per request")
    ap.add_argument("--hbm-frac", type=float, default=0.5, help="fraction of the pool the HBM tier can hold")
    ap.add_argument("--host-frac", type=float, default=1.0, help="fraction of the pool the pinned host tier can hold")
    ap.add_argument("--store-dir", default="")
    ap.add_argument("--io-backend", default="auto")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from daser_b200.config import DaserConfig
    from daser_b200.engine.rag_gpu import GpuRagEngine
    from daser_b200.models.llama import PRESETS
    from daser_b200.ops import _lib
    from daser_b200.server.__main__ import ControlPlane

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    cfg = PRESETS[args.model]
    tp_ctx = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from daser_b200.parallel.tp import TPContext

        tp_ctx = TPContext(cfg, dist.group.WORLD, max_tokens=256, impl=args.tp_impl)

    store_dir = args.store_dir or tempfile.mkdtemp(prefix="daser_bench_")
    if tp_ctx is not None:
        store_dir = tp_ctx.broadcast_object(store_dir)
    slot = cfg.num_layers * 2 * cfg.block_tokens * cfg.num_kv_heads * cfg.head_dim * 5 // 4
    prefix, pool, reqs = make_traffic(cfg.vocab_size, cfg.block_tokens, args.pool, args.k, args.steps + args.warmup)
    pool_slots = sum(len(c) // cfg.block_tokens for c in pool) + len(prefix) // cfg.block_tokens
    total_slots = pool_slots + 64
    dcfg = DaserConfig(store_path=os.path.join(store_dir, "daser.store"), index_path="", total_slots=total_slots,
                       slot_size=slot, ipc_socket_path=os.path.join(store_dir, "daser.sock"),
                       block_tokens=cfg.block_tokens, num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads,
                       head_dim=cfg.head_dim, codec="fp8b16", log_level="WARNING")
    os.environ.setdefault("DASER_LOG_LEVEL", "WARNING")

    loop = None
    if rank == 0:
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

        preallocate(dcfg.store_path, total_slots * slot)
    if tp_ctx is not None:
        tp_ctx.barrier()

    max_ctx_tokens = (args.k * 1024 + 64 + 64 + 16)
    blocks_per_req = -(-max_ctx_tokens // cfg.block_tokens)
    t0 = time.time()
    eng = GpuRagEngine(cfg, dcfg.ipc_socket_path, dcfg.store_path, num_blocks=blocks_per_req + 128, max_tokens=256,
                       max_seqs=8, hbm_slots=max(64, int(pool_slots * args.hbm_frac)),
                       host_slots=max(64, int(pool_slots * args.host_frac)) if args.host_frac > 0 else 0,
                       io_backend=args.io_backend,
                       tp_ctx=tp_ctx, staging_slots=max(blocks_per_req, 128))
    t_init = time.time() - t0

    # fill the store: real prefills through the save kernel (untimed)
    t0 = time.time()
    for c in [prefix] + pool:
        eng.store_chunk(c)
    torch.cuda.synchronize()
    t_fill = time.time() - t0

    eng.warm_up(token_counts=(64,), context_lens=(2048, 4096, 8192))

    def barrier():
        if tp_ctx is not None:
            tp_ctx.barrier()
        torch.cuda.synchronize()

    def run(req_spec):
        chunks, query, _ = req_spec
        return eng.generate(chunks, query, max_new_tokens=1)

    for spec in reqs[: args.warmup]:
        run(spec)
    eng.runner.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    from daser_b200 import metrics as _M

    pcie0 = _M.snapshot().get("connector.bytes_over_pcie", 0.0)
    barrier()
    wall0 = time.perf_counter()
    done = [run(spec) for spec in reqs[args.warmup : args.warmup + args.steps]]
    barrier()
    wall = time.perf_counter() - wall0
    launches = _lib.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else {}
    eng.runner.check_status()

    dev_ms = [r.ttft_device_ms for r in done]
    e2e_ms = [r.ttft_ms for r in done]
    restore_ms = [r.timings["restore_ms"] for r in done]
    restored_bytes = sum(r.restored_bytes for r in done)
    prompt_tokens = sum(r.context_len for r in done)
    stats = torch.tensor([percentile(dev_ms, 50), percentile(dev_ms, 99), percentile(e2e_ms, 50),
                          percentile(e2e_ms, 99), wall * 1e3 / args.steps, sum(restore_ms)], dtype=torch.float64,
                         device="cuda")
    if tp_ctx is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    p50, p99, e50, e99, ms_per_step, restore_total_ms = stats.tolist()

    if rank == 0:
        from daser_b200 import metrics as M

        snap = M.snapshot()
        io_stats = eng.worker.transfer.engine.stats()
        # per step: token ids, positions, slot mapping, block table, q_start/ctx_lens/sample rows of the
        # query prefill + the restore work list (3 int64 per slot) + the slot images the restore kernel
        # reads from pinned host memory when the chunk is not in the HBM tier
        slots_per_step = sum(r.restored_bytes for r in done) / slot / len(done)
        host_image_bytes = (snap.get("connector.bytes_over_pcie", 0.0) - pcie0) / max(args.steps, 1)
        h2d = int(64 * (4 + 4 + 8) + blocks_per_req * 4 + 3 * 4 + 8 + slots_per_step * 24 + host_image_bytes)
        out = {
            "metric": METRIC,
            "value": round(p50, 3),
            "unit": "ms",
            "n_gpus": args.gpus,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3),
            "higher_is_better": False,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic RAG traffic, random-init weights",
            "ttft_p99_ms": round(p99, 3),
            "kv_restore_gbs": round(restored_bytes / max(restore_total_ms, 1e-9) / 1e6, 2),
            "prompt_tok_s": round(prompt_tokens / wall, 1),
            "e2e": {"value": round(e50, 3), "unit": "ms", "p99": round(e99, 3), "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "config": {
                "model": cfg.name, "parallelism": f"tp{args.gpus}", "tp_impl": args.tp_impl if args.gpus > 1 else "none",
                "global_batch": 1,
                "seq_len": int(prompt_tokens / len(done)), "chunks_per_request": args.k,
                "chunk_pool": args.pool, "kv_codec": "fp8b16 (e4m3 + fp32 scale / 16)",
                "io_backend": eng.worker.transfer.backend.name, "store": dcfg.store_path,
                "tier_hits": {"hbm": int(snap.get("hbm.hits", 0)), "host": int(snap.get("host.hits", 0)),
                              "file_reads_MB": round(snap.get("connector.bytes_loaded", 0.0) / 1e6, 1)},
                "breakdown_ms_p50": {k: round(percentile([r.timings[k] for r in done], 50), 3)
                                     for k in ("plan_ms", "restore_ms", "restore_device_ms", "compute_ms")},
                "l2": "inputs larger than L2 (weights stream from HBM every step)",
                "init_s": round(t_init, 1), "fill_s": round(t_fill, 1),
                "io_direct_pieces": io_stats["direct_pieces"],
            },
        }
        print(json.dumps(out))
    eng.close()
    if rank == 0 and loop is not None:
        asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
        loop.call_soon_threadsafe(loop.stop)
    if tp_ctx is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
