"""Storage-layer benchmark: slot-sized writes, cold reads and warm reads through the transfer layer.

    python benchmarks/bench_storage.py --path /tmp/daser_bench.store --slots 100 --slot-mib 2

Counterpart of the reference's ``benchmarks/bench_storage_imdb.py`` (DaseR side): N slots of
``slot-mib`` MiB, all writes, then a cold read pass, then a warm read pass, each submitted as
one batch; throughput, per-operation p50/p95/p99 latency and a byte-equality check.  Buffers
are host memory by default, GPU memory with ``--device cuda`` (staged through pinned tiles on
host backends, DMA with GDS).  ``--backend`` picks io_uring / posix / gds explicitly.
"""

from __future__ import annotations

import argparse
import os
import time

import torch

from _common import emit, percentile

from daser_b200.connector.transfer import TransferLayer
from daser_b200.io.engine import preallocate


def drop_caches(path: str) -> None:
    """Best effort: evict the file's pages so a buffered 'cold' read is cold."""
    try:
        fd = os.open(path, os.O_RDONLY)
        os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
        os.close(fd)
    except OSError:
        pass


def run_pass(xfer, kind, bufs, slot_bytes, per_op):
    eng = xfer.engine
    t0 = time.perf_counter()
    tickets = []
    for i, b in enumerate(bufs):
        ts = time.perf_counter()
        if kind == "write":
            t = eng.submit_write(b.data_ptr(), i * slot_bytes, slot_bytes)
        else:
            t = eng.submit_read(b.data_ptr(), i * slot_bytes, slot_bytes)
        tickets.append((t, ts))
    for t, ts in tickets:
        eng.wait(t)
        per_op.append((time.perf_counter() - ts) * 1e3)
    return time.perf_counter() - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--path", default="/tmp/daser_bench.store")
    ap.add_argument("--slots", type=int, default=100)
    ap.add_argument("--slot-mib", type=float, default=2.0)
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    args = ap.parse_args()
    slot_bytes = int(args.slot_mib * (1 << 20)) // 4096 * 4096
    total = slot_bytes * args.slots
    preallocate(args.path, total)
    xfer = TransferLayer(args.path, backend=args.backend, device=0 if args.device == "cuda" else None)
    g = torch.Generator().manual_seed(0)
    if args.device == "cuda":
        src = [torch.randint(0, 255, (slot_bytes,), dtype=torch.uint8, generator=g).cuda() for _ in range(args.slots)]
        dst = [torch.empty(slot_bytes, dtype=torch.uint8, device="cuda") for _ in range(args.slots)]
        t0 = time.perf_counter()
        for i, b in enumerate(src):
            xfer.write(b, i * slot_bytes, slot_bytes)
        w = time.perf_counter() - t0
        drop_caches(args.path)
        t0 = time.perf_counter()
        for i, b in enumerate(dst):
            xfer.read_into(b, i * slot_bytes, slot_bytes)
        torch.cuda.synchronize()
        c = time.perf_counter() - t0
        t0 = time.perf_counter()
        for i, b in enumerate(dst):
            xfer.read_into(b, i * slot_bytes, slot_bytes)
        torch.cuda.synchronize()
        h = time.perf_counter() - t0
        ok = all(torch.equal(a, b) for a, b in zip(src[:5], dst[:5]))
        emit({"bench": "storage", "device": "cuda", "backend": xfer.backend.name, "slots": args.slots,
              "slot_bytes": slot_bytes, "write_GBps": total / w / 1e9, "cold_read_GBps": total / c / 1e9,
              "warm_read_GBps": total / h / 1e9, "bytes_equal": ok})
    else:
        src = [torch.randint(0, 255, (slot_bytes + 4096,), dtype=torch.uint8, generator=g) for _ in range(args.slots)]
        dst = [torch.empty(slot_bytes + 4096, dtype=torch.uint8) for _ in range(args.slots)]
        al = lambda t: t[(-t.data_ptr()) % 4096 :][:slot_bytes]  # 4 KiB aligned views (O_DIRECT eligible)
        src, dst = [al(t) for t in src], [al(t) for t in dst]
        lat = {"write": [], "cold": [], "warm": []}
        w = run_pass(xfer, "write", src, slot_bytes, lat["write"])
        drop_caches(args.path)
        c = run_pass(xfer, "read", dst, slot_bytes, lat["cold"])
        h = run_pass(xfer, "read", dst, slot_bytes, lat["warm"])
        ok = all(torch.equal(a, b) for a, b in zip(src, dst))
        row = {"bench": "storage", "device": "cpu", "backend": xfer.backend.name, "slots": args.slots,
               "slot_bytes": slot_bytes, "write_GBps": total / w / 1e9, "cold_read_GBps": total / c / 1e9,
               "warm_read_GBps": total / h / 1e9, "bytes_equal": ok, "io": xfer.engine.stats()}
        for k, v in lat.items():
            row[f"{k}_ms_p50"], row[f"{k}_ms_p95"], row[f"{k}_ms_p99"] = (percentile(v, q) for q in (50, 95, 99))
        emit(row)
    xfer.close()
    os.unlink(args.path)


if __name__ == "__main__":
    main()
