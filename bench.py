"""Headline benchmark: RAG time-to-first-token and KV-restore rate, Llama-3-70B, TP = #GPUs.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the reference arm

A *step* is one RAG request served up to its first token through the engine's public call
(``GpuRagEngine.generate``): the control plane is asked for the request's chunks; chunks in
the HBM tier are restored from there, chunks in the pinned host tier cross PCIe once, chunks in
neither are read from the store file (O_DIRECT io_uring); the fused kernel dequantises, re-rotates
keys to the chunk's new position and scatters into every rank's paged pool; the query is
prefilled over the restored context with the tcgen05 GEMMs and the fp8 paged attention; the
first token is sampled and read back.  Reads, restore pieces and the model's layers are
pipelined by layer group.

Traffic (synthetic, random-init weights; ``baseline/traffic.py``, shared with the reference arm):
a 64-token system prefix + k chunks drawn Zipf(s = 1.1) from a pool of lognormal-length chunks
(median 300 tokens, sigma 0.6, clipped to 64..1024, padded to whole 16-token blocks) + a
64-token query.  The pool (default 512 chunks) is smaller than the 20k chunks of the full
workload so that filling it (real prefills through the save kernel) fits the benchmark's time
and the box's disk; the memory tiers are sized for the head of the Zipf distribution only (HBM:
1/8 of the pool, pinned host: 1/4), so the timed requests find some chunks in each tier and some
only in the file.  All of that is printed in ``config``.

Timing: W untimed warm-up steps, then exactly K timed steps between a barrier +
``torch.cuda.synchronize()`` on both sides.  ``value`` is the p50 over the K steps of the
device-timed TTFT (CUDA events on the launching stream, max over ranks) with that tier mix;
``e2e.value`` is the p50 wall-clock TTFT of the same steps including the pinned-host -> device
copy of each step's inputs and the device -> host read of the sampled token.  After the timed
region the same engine measures, untimed for the headline: all-cold and all-warm TTFT (tiers
cleared before a request, then the same request again), the restore rate per tier, the drive's
raw read rate, and TTFT under open-loop Poisson arrivals with 128 output tokens per request.
Weights (tens of GB per GPU) are far larger than L2, so no input of a step is served from cache.
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

METRIC = "rag_ttft_p50_ms (Llama-3-70B, TP=#GPUs; chunk KV restored from the HBM tier, the host tier and the fp8 store file)"


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
        # the store (tens of GB of raw bf16 KV) lives in a directory that this process removes
        # afterwards, also when the child had to be killed
        import shutil

        made = None if args.store_dir else tempfile.mkdtemp(prefix="daser_ref_")
        cmd += ["--store-dir", args.store_dir or made]
        if os.environ.get("DASER_REF_EAGER") == "1":
            cmd.append("--eager")
        # a session of its own: on a time-out the whole group goes (vLLM's engine and worker processes too)
        proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=None, text=True, start_new_session=True)
        try:
            stdout, _ = proc.communicate(timeout=float(os.environ.get("DASER_REF_TIMEOUT", "1700")))
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
        finally:
            if made:
                shutil.rmtree(made, ignore_errors=True)
    print(json.dumps(out))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--pool", type=int, default=512, help="chunks in the synthetic pool")
    ap.add_argument("--tp-impl", choices=("auto", "fused", "twoshot", "oneshot", "nvls", "nccl"), default="auto",
                    help="auto: nvls above two GPUs where the buffers get an NVLink multicast mapping, else fused; "
                         "fused: GEMM-epilogue reduction over peer memory (one-shot all-reduce for few tokens at "
                         "tp <= 2, reduce-scatter + gated all-gather otherwise); twoshot / oneshot: force one form; "
                         "nvls: partials stay local, each rank reads the sum through the NVLink multicast mapping; "
                         "nccl: the unfused baseline (same kernels, NCCL all-reduce)")
    ap.add_argument("--k", type=int, default=8, help="chunks per request")
    ap.add_argument("--hbm-frac", type=float, default=0.125,
                    help="HBM tier of ONE rank as a fraction of the pool (the same bytes per GPU at every --gpus)")
    ap.add_argument("--host-frac", type=float, default=0.25,
                    help="pinned host tier of ONE rank as a fraction of the pool")
    ap.add_argument("--store-dir", default="")
    ap.add_argument("--io-backend", default="auto")
    ap.add_argument("--layer-groups", type=int, default=8, help="pieces the restore and the forward are pipelined in")
    ap.add_argument("--max-tokens", type=int, default=1024, help="tokens per forward (chunk fills, missed chunks)")
    ap.add_argument("--extras", type=int, default=1, help="0: skip the untimed extra measurements after the timed region")
    ap.add_argument("--open-loop-requests", type=int, default=16)
    ap.add_argument("--kv-blocks", type=int, default=6144, help="blocks of 16 tokens in the paged KV pool")
    ap.add_argument("--precondition", type=int, default=64,
                    help="untimed requests of the same traffic served before the warm-up, so that the tiers hold what "
                         "a running service's would (LRU over the Zipf traffic) instead of starting empty")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from daser_b200 import metrics as M
    from daser_b200.config import DaserConfig
    from daser_b200.engine.rag_gpu import GpuRagEngine
    from daser_b200.engine.request import RagRequest
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

        if args.tp_impl == "auto":
            # measured on the 64-token step of this model (ms, max over ranks): 2 GPUs one-shot 20.9,
            # in-switch 20.7, two-hop 22.1, NCCL 21.1; 8 GPUs in-switch 12.0, two-hop 13.1, NCCL 13.2
            tp_ctx = TPContext(cfg, dist.group.WORLD, max_tokens=args.max_tokens, impl="fused", multicast=world > 2)
            if world > 2 and tp_ctx.nv_mc:
                tp_ctx.impl = "nvls"
            args.tp_impl = tp_ctx.impl
        else:
            tp_ctx = TPContext(cfg, dist.group.WORLD, max_tokens=args.max_tokens, impl=args.tp_impl)

    store_dir = args.store_dir or tempfile.mkdtemp(prefix="daser_bench_")
    if not args.store_dir and rank == 0:
        # the store file is tens of GB: it must not outlive the run, however the run ends
        import atexit
        import shutil

        atexit.register(shutil.rmtree, store_dir, ignore_errors=True)
    elif not args.store_dir:
        os.rmdir(store_dir)  # only rank 0's directory is used
    if tp_ctx is not None:
        store_dir = tp_ctx.broadcast_object(store_dir)
    slot = cfg.num_layers * 2 * cfg.block_tokens * cfg.num_kv_heads * cfg.head_dim * 5 // 4
    # (requests are drawn one after the other: asking for more leaves the first ones as they were)
    prefix, pool, reqs = make_traffic(cfg.vocab_size, cfg.block_tokens, args.pool, args.k,
                                      args.steps + args.warmup + args.precondition
                                      + (args.open_loop_requests if args.extras else 0))
    n_timed_pre = args.steps + args.warmup + args.precondition  # then: the open-loop phase's own requests
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
    # Every GPU gives the same HBM to its tier and every rank the same pinned host memory, whatever
    # the number of ranks: a rank owns 1 / world of the chunks, so the share of the pool that fits a
    # memory tier grows with the ranks (that is what adding GPUs buys a cache).  Capped at what the
    # rank's own chunks can fill.
    own = int(pool_slots / world * 1.25) + 64
    hbm_slots = max(64, min(int(pool_slots * args.hbm_frac), own)) if args.hbm_frac > 0 else 0
    host_slots = max(64, min(int(pool_slots * args.host_frac), own)) if args.host_frac > 0 else 0
    # the paged pool holds the open-loop phase's concurrent requests (4 req/s x 128 output tokens:
    # about twenty of ~230 blocks each at TP = 1); 6144 blocks = 20 GB of fp8 KV over all ranks
    eng = GpuRagEngine(cfg, dcfg.ipc_socket_path, dcfg.store_path, num_blocks=args.kv_blocks,
                       max_tokens=args.max_tokens, max_seqs=32, hbm_slots=hbm_slots, host_slots=host_slots,
                       io_backend=args.io_backend, tp_ctx=tp_ctx, staging_slots=max(blocks_per_req, 128),
                       max_blocks=blocks_per_req + 16, layer_groups=args.layer_groups)
    t_init = time.time() - t0

    # fill the store: real prefills through the save kernel (untimed)
    t0 = time.time()
    for c in [prefix] + pool:
        eng.store_chunk(c)
    torch.cuda.synchronize()
    t_fill = time.time() - t0
    # the tiers now hold the chunks stored last; start from what the traffic makes of them
    for tier in (eng.hbm, eng.host):
        if tier is not None:
            tier.clear()

    eng.warm_up(token_counts=(64,), context_lens=(2048, 4096, 8192),
                decode_batches=(1, 2, 4, 8, 16, 32) if args.extras and args.open_loop_requests else ())

    def barrier():
        if tp_ctx is not None:
            tp_ctx.barrier()
        torch.cuda.synchronize()

    def run(req_spec):
        chunks, query, _ = req_spec
        return eng.generate(chunks, query, max_new_tokens=1)

    t0 = time.time()
    for spec in reqs[args.warmup + args.steps : n_timed_pre]:
        run(spec)
    t_precondition = time.time() - t0
    for spec in reqs[: args.warmup]:
        run(spec)
    eng.runner.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    snap0 = M.snapshot()
    io0 = eng.worker.transfer.engine.stats()
    barrier()
    wall0 = time.perf_counter()
    done = [run(spec) for spec in reqs[args.warmup : args.warmup + args.steps]]
    barrier()
    wall = time.perf_counter() - wall0
    launches = _lib.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else {}
    eng.runner.check_status()
    snap1 = M.snapshot()
    io1 = eng.worker.transfer.engine.stats()

    def delta(name):
        return snap1.get(name, 0.0) - snap0.get(name, 0.0)

    dev_ms = [r.ttft_device_ms for r in done]
    e2e_ms = [r.ttft_ms for r in done]
    restored_bytes = sum(r.restored_bytes for r in done)
    prompt_tokens = sum(r.context_len for r in done)
    # per-rank counters, summed over ranks below: tier hits, bytes read from the file, bytes over PCIe
    local = [delta("hbm.hits"), delta("host.hits"), float(io1["bytes_read"] - io0["bytes_read"]),
             float(sum(r.timings["h2d_bytes"] for r in done)), float(sum(r.timings["io_wait_ms"] for r in done))]
    stats = torch.tensor([percentile(dev_ms, 50), percentile(dev_ms, 99), percentile(e2e_ms, 50),
                          percentile(e2e_ms, 99), wall * 1e3 / args.steps], dtype=torch.float64, device="cuda")
    sums = torch.tensor(local, dtype=torch.float64, device="cuda")
    if tp_ctx is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    p50, p99, e50, e99, ms_per_step = stats.tolist()
    hbm_hits, host_hits, file_bytes, h2d_total, io_wait_total = sums.tolist()

    extras = measure_extras(args, eng, tp_ctx, reqs, barrier, rank) if args.extras else {}

    if rank == 0:
        n_loads = max(1, int(delta("connector.chunk_hits")))
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
            "ttft_ms": {"mixed_tiers": {"p50": round(p50, 3), "p99": round(p99, 3)}, **extras.get("ttft_ms", {})},
            "kv_restore_gbs": extras.get("kv_restore_gbs", {}),
            "prompt_tok_s": round(prompt_tokens / wall, 1),
            "e2e": {"value": round(e50, 3), "unit": "ms", "p99": round(e99, 3),
                    "h2d_bytes_per_step": int(h2d_total / args.steps), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "config": {
                "model": cfg.name, "parallelism": f"tp{args.gpus}", "tp_impl": args.tp_impl if args.gpus > 1 else "none",
                "global_batch": 1,
                "seq_len": int(prompt_tokens / len(done)), "chunks_per_request": args.k,
                "chunk_pool": args.pool,
                "chunk_pool_note": "20k in the full workload; scaled so that the fill (a real prefill and save per chunk) "
                                   "fits the run; tiers are sized relative to the pool",
                "kv_codec": "fp8b16 (e4m3 + fp32 scale / 16)",
                "io_backend": eng.worker.transfer.backend.name, "store": dcfg.store_path,
                "tiers": {"hbm_slots_per_rank": hbm_slots, "host_slots_per_rank": host_slots, "pool_slots": pool_slots,
                          "owner": "hash(chunk_key) mod tp",
                          "sizing": "the same bytes per rank at every N (a rank owns 1/N of the chunks, so the "
                                    "tiers of N ranks together hold N times the share of the pool)",
                          "share_of_pool": {"hbm": round(min(1.0, hbm_slots * world / pool_slots), 3),
                                            "host": round(min(1.0, host_slots * world / pool_slots), 3)}},
                "tier_hits": {"hbm": int(hbm_hits), "host": int(host_hits),
                              "file": int(delta("connector.chunk_hits") - hbm_hits - host_hits),
                              "file_reads_MB": round(file_bytes / 1e6, 1),
                              "restored_MB": round(restored_bytes / 1e6, 1),
                              "io_wait_ms_per_step": round(io_wait_total / args.steps / max(world, 1), 3)},
                "breakdown_ms_p50": {k: round(percentile([r.timings[k] for r in done], 50), 3)
                                     for k in ("plan_ms", "restore_ms", "compute_ms", "io_wait_ms")},
                "pipeline": f"{len(eng.runner.layer_groups)} layer groups: reads, restore pieces and layers overlap",
                "arrivals": "closed loop, one request at a time (value); open loop under config.open_loop",
                "open_loop": extras.get("open_loop", {}),
                "l2": "inputs larger than L2 (weights stream from HBM every step)",
                "init_s": round(t_init, 1), "fill_s": round(t_fill, 1),
                "tier_precondition": f"{args.precondition} untimed requests of the same traffic served after the fill "
                                     f"(tiers emptied first) and before the warm-up, {round(t_precondition, 1)} s: the "
                                     "tiers hold what LRU makes of the Zipf traffic, not an empty cache",
                "io_direct_pieces": io1["direct_pieces"],
            },
        }
        print(json.dumps(out))
    eng.close()
    if rank == 0 and loop is not None:
        asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
        loop.call_soon_threadsafe(loop.stop)
    if tp_ctx is not None:
        dist.destroy_process_group()


def measure_extras(args, eng, tp_ctx, reqs, barrier, rank) -> dict:
    """Untimed for the headline, on the engine that just ran it: all-cold and all-warm TTFT, the
    restore rate out of each tier, the drive's raw read rate, TTFT under open-loop arrivals."""
    import torch
    import torch.distributed as dist

    from daser_b200.connector.core import ConnectorMeta
    from daser_b200.engine.request import RagRequest
    from daser_b200.hashing import hash_tokens

    world = eng.tp
    tiers = [t for t in (eng.hbm, eng.host) if t is not None]

    def reduce_max(vals):
        t = torch.tensor(vals, dtype=torch.float64, device="cuda")
        if tp_ctx is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # ---- all-cold, then the same request again: all-warm ----
    sample = reqs[args.warmup : args.warmup + min(args.steps, 8)]
    cold, warm = [], []
    for chunks, query, _ in sample:
        for t in tiers:
            t.clear()
        barrier()
        cold.append(eng.generate(chunks, query, max_new_tokens=1).ttft_device_ms)
        barrier()
        warm.append(eng.generate(chunks, query, max_new_tokens=1).ttft_device_ms)
    c50, c99, w50, w99 = reduce_max([percentile(cold, 50), percentile(cold, 99), percentile(warm, 50), percentile(warm, 99)])
    out = {"ttft_ms": {"all_cold_file": {"p50": round(c50, 3), "p99": round(c99, 3), "requests": len(sample)},
                       "all_warm_tiers": {"p50": round(w50, 3), "p99": round(w99, 3), "requests": len(sample)}}}

    # ---- restore rate per tier: one request's chunks, unpipelined, device-timed on this rank ----
    chunks, query, _ = sample[0]
    bt = eng.cfg.block_tokens
    placements, pos = [], 0
    for c in chunks:
        placements.append((hash_tokens(c), pos))
        pos += len(c)
    table = eng.blocks.alloc(pos // bt)
    rates = {}
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for name in ("file", "host", "hbm"):
        meta = None
        if eng.sched is not None:
            eng.sched.plan_chunk_loads("probe-" + name, placements)
            eng.sched.assign_chunk_blocks("probe-" + name, table)
            meta = eng.sched.build_connector_meta(["probe-" + name])
            eng.sched.request_finished("probe-" + name)
        meta = eng._bcast(meta)
        mine = ConnectorMeta(reqs_to_load=[s for s in meta.reqs_to_load if eng.owner_of(s.chunk_key) == eng.rank])
        if name == "file":
            for t in tiers:
                t.clear()
        elif name == "host" and eng.hbm is not None:
            eng.hbm.clear()
        nbytes = sum(len(s.block_ids) for s in mine.reqs_to_load) * eng.geo.slot_size
        barrier()
        ev[0].record()
        ticket = eng.worker.begin_load(mine)
        if ticket is not None:
            eng.worker.restore_group(ticket, 0)
            eng.worker.end_load(ticket, wait=True)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1])  # spans the host's wait for the reads too: the GPU idles meanwhile
        barrier()
        tb = ticket.tier_bytes if ticket is not None else {}
        src = [tb.get("hbm", 0), tb.get("host", 0), tb.get("host_fill", 0) + tb.get("staging", 0)]
        agg = torch.tensor([float(nbytes), ms] + [float(b) for b in src], dtype=torch.float64, device="cuda")
        if tp_ctx is not None:
            parts = [torch.zeros_like(agg) for _ in range(world)]
            dist.all_gather(parts, agg)
            total_bytes = sum(p[0].item() for p in parts)
            slowest = max(p[1].item() for p in parts)
            src = [sum(p[2 + i].item() for p in parts) for i in range(3)]
        else:
            total_bytes, slowest = nbytes, ms
        rates[f"restore_{name}_gbs"] = round(total_bytes / max(slowest, 1e-6) / 1e6, 2)
        rates[f"restore_{name}_ms"] = round(slowest, 3)
        # where the bytes really came from (a rank whose tier is smaller than its share of the
        # request falls through to the next source)
        rates[f"restore_{name}_sources_MB"] = {k: round(b / 1e6, 1) for k, b in zip(("hbm", "host", "file"), src)}
    eng.blocks.free(table)
    rates["note"] = ("one request's chunks, all ranks restoring their own at once, no pipelining, device + host timed, "
                     "max over ranks: file = store file -> pinned host tier -> HBM tier -> pools; host = pinned host "
                     "tier -> HBM tier -> pools; hbm = HBM tier -> pools (the fused kernel alone)")
    # the drive itself: a sequential read of up to 2 GiB of the store through the same IO engine
    io = eng.worker.transfer.engine
    probe = eng.worker._staging
    n = min(probe.numel(), 2 << 30, io.file_size) // (1 << 20) * (1 << 20)
    if not probe.is_cuda and n > 0 and rank == 0:
        t0 = time.perf_counter()
        io.wait(io.submit_read(probe.data_ptr(), 0, n))
        rates["drive_read_gbs"] = round(n / (time.perf_counter() - t0) / 1e9, 2)
        if rates.get("restore_file_ms"):
            rates["restore_file_vs_drive"] = round(rates["restore_file_gbs"] / rates["drive_read_gbs"], 2)
    barrier()
    out["kv_restore_gbs"] = rates

    # ---- open loop: Poisson arrivals at 4 req/s, 128 output tokens each, TTFT from arrival ----
    n_open = args.open_loop_requests
    if n_open > 0:
        import random

        # the probes above emptied the tiers: bring them back to what the traffic makes of them
        for t in tiers:
            t.clear()
        n_pre = args.warmup + args.steps + args.precondition
        for chunks, query, _ in reqs[args.warmup + args.steps : n_pre]:
            eng.generate(chunks, query, max_new_tokens=1)

        rng = random.Random(7)
        gaps = [rng.expovariate(4.0) for _ in range(n_open)]
        picks = reqs[n_pre : n_pre + n_open]  # requests nobody has served yet: the tier mix of the headline
        barrier()
        t_begin = time.perf_counter()
        arrivals, t = [], 0.0
        for g in gaps:
            t += g
            arrivals.append(t)
        pending = list(zip(arrivals, picks))
        live = []
        while pending or eng.waiting or eng.running:
            # rank 0's clock decides how many requests have arrived; every rank submits the same ones
            due = 0
            if rank == 0:
                now = time.perf_counter() - t_begin
                if pending and not (eng.waiting or eng.running) and pending[0][0] > now:
                    time.sleep(min(0.002, pending[0][0] - now))
                    now = time.perf_counter() - t_begin
                due = sum(1 for at, _ in pending if at <= now)
            due = eng._bcast(due)
            for _ in range(due):
                at, (chunks, query, _) = pending.pop(0)
                r = RagRequest([list(c) for c in chunks], list(query), 128)
                r.arrival = t_begin + at
                live.append(eng.submit(r))
            if eng.waiting or eng.running:
                eng.step()
        barrier()
        ttft = [(r.first_token_time - r.arrival) * 1e3 for r in live if getattr(r, "first_token_time", 0)]
        span = time.perf_counter() - t_begin
        if ttft:
            o50, o99 = reduce_max([percentile(ttft, 50), percentile(ttft, 99)])
            out["open_loop"] = {"arrivals": "Poisson 4 req/s", "requests": n_open, "output_tokens": 128,
                                "ttft_from_arrival_ms": {"p50": round(o50, 3), "p99": round(o99, 3)},
                                "output_tok_s": round(sum(len(r.generated) for r in live) / span, 1)}
    return out


if __name__ == "__main__":
    main()
