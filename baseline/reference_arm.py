"""The reference arm of the headline benchmark: the unmodified reference (installed under
``baseline/_ref``) inside the stock ``vllm.LLM``, serving the same synthetic RAG requests.

How the reference reuses KV: only an identical prompt prefix can hit
(``daser/retrieval/prefix.py:49-72``), so, exactly as in its own end-to-end benchmark
(``benchmarks/bench_e2e_daser_vs_lmcache.py:404-466``), every request is first served cold
(prefill, store to the file, commit) and then served again with the identical prompt; the
second, warm pass is the timed one.  The control plane is the reference's own ``IPCServer`` on
a thread (``benchmarks/bench_e2e_daser_vs_lmcache.py:236-266``); the connector is loaded by
vLLM through ``kv_connector_module_path``.  ``kvikio`` and ``cupy`` come from the stand-ins under
``baseline/shims`` (kvikio's compatibility mode: POSIX IO on a thread pool through a pinned
bounce buffer), since neither wheel exists offline.

The time to first token is the wall-clock time of ``LLM.generate`` with ``max_tokens=1`` on one
request at a time: it includes the host-to-device copy of the prompt and the device-to-host
read of the sampled token, so it is an end-to-end number.

Run by ``bench.py --impl reference`` in a process of its own whose environment carries no
launcher variables; prints one JSON line.
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
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

from traffic import MODEL_SHAPES, make_traffic, percentile  # noqa: E402
import vllm_common as vc  # noqa: E402

METRIC = "rag_ttft_p50_ms (Llama-3-70B, TP=#GPUs)"
BLOCK_TOKENS = 16


class ReferenceControlPlane:
    """The reference's control plane on a daemon thread, wired as its own harnesses wire it."""

    def __init__(self, tmpdir: str, total_slots: int, slot_size: int) -> None:
        self.socket_path = os.path.join(tmpdir, "daser.sock")
        self.store_path = os.path.join(tmpdir, "daser.store")
        self.total_slots, self.slot_size = total_slots, slot_size
        self._loop = None
        self._server = None

    def start(self) -> None:
        from daser.position.fixed_offset import FixedOffsetEncoder
        from daser.retrieval.prefix import PrefixHashIndex
        from daser.server.chunk_manager import ChunkManager
        from daser.server.ipc_server import IPCServer
        from daser.server.metadata_store import MetadataStore

        with open(self.store_path, "wb") as f:
            f.truncate(self.total_slots * self.slot_size)
        metadata = MetadataStore(total_slots=self.total_slots)
        cm = ChunkManager(total_slots=self.total_slots, metadata_store=metadata)
        server = IPCServer(socket_path=self.socket_path, chunk_manager=cm,
                           retrieval_index=PrefixHashIndex(block_tokens=BLOCK_TOKENS),
                           position_encoder=FixedOffsetEncoder(fixed_offset=0), slot_size=self.slot_size,
                           block_tokens=BLOCK_TOKENS)
        loop = asyncio.new_event_loop()
        started = threading.Event()

        def run() -> None:
            asyncio.set_event_loop(loop)
            loop.run_until_complete(server.start())
            started.set()
            loop.run_forever()

        threading.Thread(target=run, daemon=True, name="daser-ref-server").start()
        if not started.wait(10.0):
            raise RuntimeError("reference IPCServer did not start")
        self._loop, self._server = loop, server

    def stop(self) -> None:
        if self._server is not None:
            try:
                asyncio.run_coroutine_threadsafe(self._server.stop(), self._loop).result(10.0)
            except Exception:  # noqa: BLE001
                pass
            self._loop.call_soon_threadsafe(self._loop.stop)


def run(args) -> dict:
    shape = MODEL_SHAPES[args.model]
    tp = args.gpus
    n_req = args.steps + args.warmup
    prefix, pool, reqs = make_traffic(shape["vocab_size"], BLOCK_TOKENS, args.pool, args.k, n_req)
    # the prompt must not be a whole number of blocks: a full-prompt hit leaves vLLM nothing to
    # schedule (it asserts num_new_tokens > 0), so the last query token is dropped
    prompts = [[t for c in chunks for t in c] + query[:-1] for chunks, query, _ in reqs]
    max_len = max(len(p) for p in prompts) + 16
    max_model_len = -(-max_len // 1024) * 1024

    # the reference is not rank-aware: every tensor-parallel rank reads and writes the same file
    # offsets (daser/connector/daser_connector.py:150-156, 652).  The slot is sized for ONE rank's
    # heads, the cheapest consistent choice for it; restored KV at tp > 1 is whatever rank wrote
    # last, so tp > 1 numbers are timing only.
    slot = vc.slot_size_bf16(args.model, BLOCK_TOKENS, tp)
    need_slots = sum(-(-len(p) // BLOCK_TOKENS) for p in prompts) + 64
    tmpdir = args.store_dir or tempfile.mkdtemp(prefix="daser_ref_")
    free = shutil.disk_usage(tmpdir).free
    if need_slots * slot > free * 0.9:
        raise RuntimeError(f"store of {need_slots * slot >> 20} MiB does not fit {tmpdir} ({free >> 20} MiB free)")
    plane = ReferenceControlPlane(tmpdir, need_slots, slot)
    plane.start()
    model_dir = vc.write_hf_config(args.model, os.path.join(tmpdir, "model"))
    ktc = {
        "kv_connector": "DaserConnector",
        "kv_connector_module_path": "daser.connector.daser_connector",
        "kv_role": "kv_both",
        "kv_connector_extra_config": {"socket_path": plane.socket_path, "store_path": plane.store_path,
                                      "slot_size": slot, "block_tokens": BLOCK_TOKENS, "model_id": args.model},
    }
    t0 = time.time()
    llm = vc.build_llm(model_dir, tp, ktc, max_model_len, gpu_memory_utilization=args.gpu_util,
                       attention_backend="FLASH_ATTN", enforce_eager=args.eager)
    init_s = time.time() - t0
    try:
        vc.first_token_ms(llm, [5] * 40)  # untimed first call; shares no block with any prompt, so it cannot become a prefix hit
        t0 = time.time()
        cold = [vc.first_token_ms(llm, p) for p in prompts]  # miss: prefill + store + commit
        cold_s = time.time() - t0
        for p in prompts[: args.warmup]:
            vc.first_token_ms(llm, p)
        sampler = vc.ClockSampler(0)
        sampler.start()
        wall0 = time.perf_counter()
        warm = [vc.first_token_ms(llm, p) for p in prompts[args.warmup :]]  # hit: read + scatter + tail
        wall = time.perf_counter() - wall0
        clocks = sampler.stop()
    finally:
        vc.destroy_llm(llm)
        plane.stop()
    warm_ms = [m for m, _ in warm]
    cold_ms = [m for m, _ in cold[args.warmup :]]
    mismatches = sum(1 for (_, a), (_, b) in zip(cold[args.warmup :], warm) if a != b)
    timed = prompts[args.warmup :]
    prompt_tokens = sum(len(p) for p in timed)
    restored_bytes = sum((len(p) // BLOCK_TOKENS) * slot * tp for p in timed)
    p50 = percentile(warm_ms, 50)
    out = {
        "impl": "reference",
        "reference_class": "unmodified reference connector + control plane in stock vllm.LLM; kvikio/cupy replaced by "
                           "compat-mode stand-ins (POSIX thread pool + pinned bounce buffer)",
        "metric": METRIC, "value": round(p50, 3), "unit": "ms", "n_gpus": tp, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(wall * 1e3 / max(len(timed), 1), 3), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic RAG traffic, random-init weights (load_format=dummy)",
        "ttft_p99_ms": round(percentile(warm_ms, 99), 3),
        "cold_ttft_p50_ms": round(percentile(cold_ms, 50), 3),
        "kv_restore_gbs": round(restored_bytes / (sum(warm_ms) / 1e3) / 1e9, 3),
        "prompt_tok_s": round(prompt_tokens / wall, 1),
        "e2e": {"value": round(p50, 3), "unit": "ms", "p99": round(percentile(warm_ms, 99), 3),
                "h2d_bytes_per_step": int(prompt_tokens / len(timed) * 8 + restored_bytes / len(timed)),
                "d2h_bytes_per_step": 8},
        "timing": "wall clock around LLM.generate(max_tokens=1), one request at a time (device timing is not "
                  "reachable from outside the engine process); kv_restore_gbs = restored KV bytes / warm TTFT",
        "clocks": clocks,
        "config": {
            "model": args.model, "parallelism": f"tp{tp}", "global_batch": 1,
            "seq_len": int(prompt_tokens / len(timed)), "chunks_per_request": args.k, "chunk_pool": args.pool,
            "kv_codec": "raw bf16", "io_backend": "kvikio compat (stand-in), buffered POSIX, 4 threads",
            "attention_backend": "FLASH_ATTN (forced: the reference indexes that KV layout)",
            "hit_mode": "identical prompt replayed (cold pass stores, warm pass timed)",
            "cold_vs_warm_first_token_mismatches": f"{mismatches}/{len(warm)}",
            "tp_note": "tp > 1 is timing only: the reference's ranks share file offsets" if tp > 1 else "",
            "enforce_eager": bool(args.eager), "init_s": round(init_s, 1), "cold_pass_s": round(cold_s, 1),
            "slot_size": slot, "store_MB": need_slots * slot >> 20,
            "l2": "inputs larger than L2 (weights stream from HBM every step)",
        },
    }
    if not args.store_dir:
        shutil.rmtree(tmpdir, ignore_errors=True)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--pool", type=int, default=512)
    ap.add_argument("--k", type=int, default=8)
    ap.add_argument("--gpu-util", type=float, default=0.92)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--store-dir", default="")
    args = ap.parse_args()
    try:
        out = run(args)
    except BaseException as exc:  # noqa: BLE001
        traceback.print_exc()
        out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    print("REFERENCE_RESULT " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
