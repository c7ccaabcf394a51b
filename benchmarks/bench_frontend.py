"""The HTTP front end of the in-process engine, on the CPU engine (no GPU): what a client sees.

    python benchmarks/bench_frontend.py [--long-tokens 150] [--short 6]

Starts ``python -m daser_b200.service --engine native`` twice, without and with ``--native-batching``,
and for each: one long streamed request is started, and while it generates, ``--short`` short requests
arrive one after the other.  Reported per mode: the streamed time to first token of the long request,
and the time to first token of the short ones (median, worst).  Without the engine loop a short
request waits for the long one to finish; with it, its prefill runs between two decode steps.
The toy model on CPU makes a step cost milliseconds: the figures show the scheduling, not a GPU.
(The service runs with ``OMP_NUM_THREADS=1``: PyTorch keeps one OpenMP pool per calling Python thread,
and the pools of the thread that built the engine and of the thread that steps it otherwise spin
against each other, which made the engine loop look 2.7 times slower per step on this CPU model.)
The reference has no front end of its own to compare with (it forwards to a remote vLLM).
"""

from __future__ import annotations

import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import tempfile
import threading
import time
import urllib.request

from _common import ROOT, emit, percentile


def _post_stream(base, body):
    """(time to first event, total time) of one streamed completion."""
    req = urllib.request.Request(base + "/v1/completions", data=json.dumps(dict(body, stream=True)).encode(),
                                 headers={"content-type": "application/json"})
    t0 = time.perf_counter()
    first = None
    with urllib.request.urlopen(req, timeout=600) as r:
        for raw in r:
            if raw.startswith(b"data: {") and first is None:
                first = time.perf_counter() - t0
    return first, time.perf_counter() - t0


def run_mode(batching: bool, args) -> dict:
    tmp = tempfile.mkdtemp(prefix="daser_fe_")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "daser_b200.service", "--engine", "native", "--tokenizer", "byte", "--store-path",
           f"{tmp}/s.store", "--index-path", f"{tmp}/s.index", "--socket-path", f"{tmp}/s.sock", "--total-slots", "256",
           "--host", "127.0.0.1", "--port", str(port)] + (["--native-batching"] if batching else [])
    proc = subprocess.Popen(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, cwd=ROOT,
                            env=dict(os.environ, DASER_LOG_LEVEL="WARNING", OMP_NUM_THREADS="1"))
    base = f"http://127.0.0.1:{port}"
    try:
        deadline = time.time() + 60
        while True:
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    if json.load(r)["status"] == "ok":
                        break
            except OSError:
                if time.time() > deadline or proc.poll() is not None:
                    raise SystemExit("service did not start")
                time.sleep(0.2)
        _post_stream(base, {"prompt": [1, 2, 3], "max_tokens": 2})  # warm-up
        long_result = {}
        t = threading.Thread(target=lambda: long_result.update(
            zip(("ttft", "total"), _post_stream(base, {"prompt": list(range(1, 40)), "max_tokens": args.long_tokens}))))
        t.start()
        time.sleep(0.15)  # the long request is generating by now
        short = []
        for i in range(args.short):
            short.append(_post_stream(base, {"prompt": [7 + i] * 20, "max_tokens": 2})[0] * 1e3)
        t.join()
        return {"bench": "frontend", "batching": batching, "long_tokens": args.long_tokens,
                "long_ttft_ms": long_result["ttft"] * 1e3, "long_total_ms": long_result["total"] * 1e3,
                "short_ttft_ms_p50": percentile(short, 50), "short_ttft_ms_max": max(short)}
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(30)
        except subprocess.TimeoutExpired:
            proc.kill()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--long-tokens", type=int, default=150)
    ap.add_argument("--short", type=int, default=6)
    args = ap.parse_args()
    for batching in (False, True):
        emit(run_mode(batching, args))


if __name__ == "__main__":
    main()
