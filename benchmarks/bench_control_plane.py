"""Control-plane micro-benchmark: RPC round trips and index lookups (CPU only, no GPU).

    python benchmarks/bench_control_plane.py [--chunks 2000] [--clients 8] [--prompt-tokens 4096]

A control plane is started as a separate process (``python -m daser_b200.server``), filled with
``--chunks`` committed chunks, and driven over its Unix socket:

* one client: latency of ``lookup`` (longest-prefix over a ``--prompt-tokens`` prompt),
  ``lookup_chunks`` (8 keys, the RAG plan of one request) and an ``alloc_chunk`` + ``commit_chunk``
  pair; p50 / p99 over ``--iters`` calls;
* ``--clients`` concurrent client processes: ``lookup_chunks`` calls per second, against the Python
  server and against the native lookup thread (``server/csrc/fast_lookup.cc``).

In-process figures for comparison: the longest-prefix lookup with the native index and with the
pure-Python path (what the reference's algorithm costs is the third line: re-hashing every
candidate prefix from scratch, ``daser/retrieval/prefix.py:63-72``).
The reference publishes no control-plane numbers.
"""

from __future__ import annotations

import argparse
import os
import random
import signal
import subprocess
import sys
import tempfile
import threading
import time

from _common import ROOT, emit, percentile

from daser_b200 import hashing
from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.retrieval.prefix import PrefixHashIndex
from daser_b200.server import native_index
from daser_b200.server.metadata_store import ChunkMeta

SLOT = 4096


def _timed(fn, iters):
    out = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        out.append((time.perf_counter() - t0) * 1e6)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--chunks", type=int, default=2000)
    ap.add_argument("--clients", type=int, default=8)
    ap.add_argument("--prompt-tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=300)
    args = ap.parse_args()
    rng = random.Random(0)
    tmp = tempfile.mkdtemp(prefix="daser_cp_")
    sock = os.path.join(tmp, "d.sock")
    total_slots = args.chunks * 4 + 1024
    proc = subprocess.Popen(
        [sys.executable, "-m", "daser_b200.server", "--store-path", os.path.join(tmp, "d.store"), "--store-size",
         str(total_slots * SLOT), "--socket-path", sock, "--index-path", os.path.join(tmp, "d.index"), "--slot-size",
         str(SLOT), "--model-id", "m", "--log-level", "WARNING"],
        stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, cwd=ROOT)
    try:
        deadline = time.time() + 60
        while not os.path.exists(sock):
            if time.time() > deadline or proc.poll() is not None:
                raise SystemExit("control plane did not start")
            time.sleep(0.05)
        client = IPCClientSync(sock)
        # fill: chunks of 64 tokens; the long prompt's 1024-token prefix is one of them
        prompt = [rng.randrange(128000) for _ in range(args.prompt_tokens)]
        keys = []
        t0 = time.perf_counter()
        for i in range(args.chunks):
            toks = prompt[:1024] if i == 0 else [rng.randrange(128000) for _ in range(64)]
            key = hashing.hash_tokens(toks)
            client.alloc_chunk(key, len(toks), "m")
            client.commit_chunk(key)
            keys.append(key)
        fill_s = time.perf_counter() - t0
        emit({"bench": "control_plane", "what": "fill (alloc + commit per chunk)", "chunks": args.chunks,
              "chunks_per_s": args.chunks / fill_s})

        lat = _timed(lambda: client.lookup(prompt, "m"), args.iters)
        emit({"bench": "control_plane", "what": f"lookup RPC, {args.prompt_tokens}-token prompt (hit at 1024), "
              "token ids as a msgpack list (the reference's wire form)",
              "p50_us": percentile(lat, 50), "p99_us": percentile(lat, 99)})
        packed = IPCClientSync(sock)
        if packed.negotiate():
            lat = _timed(lambda: packed.lookup(prompt, "m"), args.iters)
            emit({"bench": "control_plane", "what": f"lookup RPC, {args.prompt_tokens}-token prompt, "
                  "token ids as packed int32 (negotiated)", "p50_us": percentile(lat, 50), "p99_us": percentile(lat, 99)})
        packed.close()
        plan = lambda: client.lookup_chunks(rng.sample(keys, 8), "m")  # noqa: E731
        lat = _timed(plan, args.iters)
        emit({"bench": "control_plane", "what": "lookup_chunks RPC, 8 keys", "p50_us": percentile(lat, 50),
              "p99_us": percentile(lat, 99)})
        scan = IPCClientSync(sock)
        scan.negotiate()
        for label, extra in (("block-aligned offsets", {}), ("every token offset", {"any_offset": True})):
            msg = {"op": "lookup_chunks", **scan._tok(prompt), "model_id": "m", **extra}
            lat = _timed(lambda: scan.call(msg), max(20, args.iters // 5))
            emit({"bench": "control_plane", "what": f"lookup_chunks scan RPC, {args.prompt_tokens}-token prompt, "
                  f"{label} (the completions route runs the second per request)", "p50_us": percentile(lat, 50),
                  "p99_us": percentile(lat, 99)})
        scan.close()
        native = IPCClientSync(sock)
        native.negotiate()
        has_native = getattr(native, "_fast", None) is not None
        if has_native:
            lat = _timed(lambda: native.lookup_chunks(rng.sample(keys, 8), "m"), args.iters)
            emit({"bench": "control_plane", "what": "lookup_chunks RPC, 8 keys, native lookup thread",
                  "p50_us": percentile(lat, 50), "p99_us": percentile(lat, 99)})
        native.close()
        n = [0]

        def alloc_commit():
            n[0] += 1
            key = hashing.hash_tokens([n[0]] * 16)
            client.alloc_chunk(key, 16, "m")
            client.commit_chunk(key)

        lat = _timed(alloc_commit, args.iters)
        emit({"bench": "control_plane", "what": "alloc_chunk + commit_chunk RPC pair", "p50_us": percentile(lat, 50),
              "p99_us": percentile(lat, 99)})

        # concurrent clients are processes (threads of one interpreter would measure its lock)
        for label, use_native in (("python server", False), ("native lookup thread", True)):
            if use_native and not has_native:
                continue
            code = (
                "import sys, time, random\n"
                "from daser_b200.connector.ipc_client import IPCClientSync\n"
                "sock, seed, native = sys.argv[1], int(sys.argv[2]), sys.argv[3] == '1'\n"
                "keys = sys.stdin.read().split()\n"
                "c = IPCClientSync(sock)\n"
                "if native: c.negotiate()\n"
                "r = random.Random(seed); n = 0; stop = time.time() + 3.0\n"
                "while time.time() < stop:\n"
                "    c.lookup_chunks(r.sample(keys, 8), 'm'); n += 1\n"
                "print(n)\n"
            )
            procs = [subprocess.Popen([sys.executable, "-c", code, sock, str(i), "1" if use_native else "0"],
                                      stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
                     for i in range(args.clients)]
            for p in procs:
                p.stdin.write(" ".join(keys))
                p.stdin.close()
            total = sum(int(p.stdout.read().strip() or 0) for p in procs)
            for p in procs:
                p.wait()
            emit({"bench": "control_plane", "what": f"lookup_chunks RPC, {args.clients} concurrent client "
                  f"processes, {label}", "calls_per_s": total / 3.0})
        client.close()
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(20)
        except subprocess.TimeoutExpired:
            proc.kill()

    # in process: the index alone
    import asyncio

    loop = asyncio.new_event_loop()
    for label, native in (("native index", True), ("python index", False)):
        if native and not native_index.available():
            continue
        ix = PrefixHashIndex(16, native=native)
        loop.run_until_complete(ix.insert(ChunkMeta(hashing.hash_tokens(prompt[:1024]), 0, 64, 1024, 0, "m")))
        lat = _timed(lambda: ix.lookup_sync(prompt, "m"), 200)
        emit({"bench": "index", "what": f"longest-prefix lookup, {args.prompt_tokens} tokens, {label}",
              "p50_us": percentile(lat, 50)})

    def quadratic():
        for nb in range(len(prompt) // 16, 0, -1):
            if hashing.hash_tokens(prompt[: nb * 16]) == keys[0]:
                return nb

    lat = _timed(quadratic, 5)
    emit({"bench": "index", "what": f"longest-prefix lookup, {args.prompt_tokens} tokens, re-hash every prefix "
          "(the reference's algorithm)", "p50_us": percentile(lat, 50)})


if __name__ == "__main__":
    main()
