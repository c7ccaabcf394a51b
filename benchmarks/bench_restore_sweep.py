"""Storage / restore sweep with no model: NVMe rate, scatter rate and end-to-end restore latency.

    python benchmarks/bench_restore_sweep.py                      # 1 GPU, TP shards emulated on it
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_restore_sweep.py                          # N GPUs, real peer pools

Synthetic KV chunks of 64..4096 tokens x 80 layers x 8 KV heads x 128 dims (bf16 source values
N(0, 0.5), block-scaled fp8 on disk) are compressed and written through the storage engine, then
restored into tensor-parallel-sharded paged pools with RoPE re-rotation to random offsets by the
fused kernel running on rank 0 (peer stores over NVLink when N > 1).  Per chunk size it reports
  * store-file write and read GB/s (the NVMe leg, O_DIRECT, against nothing but itself: the
    drive's own rate on this box is whatever these two lines say),
  * the scatter kernel's GB/s from HBM-resident images (the NVLink / HBM leg) and its fraction of
    the roofline (slower of HBM traffic on rank 0 and bytes leaving over NVLink at 770 GB/s),
  * the end-to-end restore latency file -> pinned host -> pools.
"""

from __future__ import annotations

import argparse
import os
import random
import tempfile
import time

import torch
import torch.distributed as dist

from _common import emit, peaks, time_cuda

from daser_b200.connector.transfer import TransferLayer
from daser_b200.io.engine import preallocate
from daser_b200.kv.layout import KVGeometry
from daser_b200.ops import kv_ops
from daser_b200.position import inv_freq_table

NVLINK_GBS = 770.0  # measured peer copy rate per direction on this pool


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="64,256,1024,4096")
    ap.add_argument("--tp", type=int, default=8, help="shards to emulate when run on one GPU")
    ap.add_argument("--dir", default="")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    geo = KVGeometry(80, 8, 128, 16, 2, "fp8b16")
    sizes = [int(s) for s in args.sizes.split(",")]
    max_slots = max(sizes) // 16
    n_blocks = max_slots + 16
    tp = world if world > 1 else args.tp
    hn = 8 // tp
    shape = (80, n_blocks, 2, hn, 16, 128)
    ctx = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        import torch.distributed._symmetric_memory as symm

        pay = symm.empty(shape, dtype=torch.uint8, device="cuda")
        sc = symm.empty(shape[:-1] + (8,), dtype=torch.float32, device="cuda")
        h1, h2 = symm.rendezvous(pay, dist.group.WORLD.group_name), symm.rendezvous(sc, dist.group.WORLD.group_name)
        pool = kv_ops.PagedKVPool(
            payload_ptrs=[int(p) for p in h1.buffer_ptrs], scale_ptrs=[int(p) for p in h2.buffer_ptrs],
            stride_layer=pay.stride(0), stride_block=pay.stride(1), stride_kv=pay.stride(2), stride_tok=pay.stride(4),
            stride_head=pay.stride(3), num_blocks=n_blocks, heads_per_rank=hn, is_fp8=True, keepalive=[pay, sc])
        ctx = True
    else:
        pays = [torch.zeros(shape, dtype=torch.uint8, device="cuda") for _ in range(tp)]
        scs = [torch.zeros(shape[:-1] + (8,), dtype=torch.float32, device="cuda") for _ in range(tp)]
        pool = kv_ops.PagedKVPool.from_tensors(pays, scs, "LNKHTD")
    hbm, _, kind = peaks()
    if rank == 0:
        d = args.dir or tempfile.mkdtemp(prefix="daser_sweep_")
        path = os.path.join(d, "sweep.store")
        preallocate(path, max_slots * geo.slot_size)
        xfer = TransferLayer(path, backend="auto", device=None)
        host = torch.empty(max_slots * geo.slot_size, dtype=torch.uint8).pin_memory()
        dev_img = torch.empty(max_slots * geo.slot_size, dtype=torch.uint8, device="cuda")
        cos_sin = kv_ops.rope_table(32768, inv_freq_table(128, 500000.0), "cuda")
        status = torch.zeros(2, dtype=torch.int32, device="cuda")
        rng = random.Random(0)
    for tokens in sizes:
        n = tokens // 16
        if rank == 0:
            # source KV N(0, 0.5) in a single-rank bf16 pool -> fp8b16 slot images with the save kernel
            src = (torch.randn(80, n, 2, 8, 16, 128, device="cuda") * 0.5).to(torch.bfloat16)
            src_pool = kv_ops.PagedKVPool.from_tensors([src], None, "LNKHTD")
            work_s = kv_ops.KVWorkList(
                torch.tensor([dev_img.data_ptr() + i * geo.slot_size for i in range(n)], dtype=torch.int64, device="cuda"),
                torch.arange(n, dtype=torch.int32, device="cuda"))
            save_ms, _ = time_cuda(lambda: kv_ops.kv_save(work_s, geo, src_pool, 0, status), iters=5)
            nbytes = n * geo.slot_size
            host[:nbytes].copy_(dev_img[:nbytes])
            torch.cuda.synchronize()
            eng = xfer.engine
            t0 = time.perf_counter()
            eng.wait(eng.submit_write(host.data_ptr(), 0, nbytes))
            w_s = time.perf_counter() - t0
            blocks = torch.randperm(n_blocks)[:n].to(torch.int32).cuda()
            deltas = torch.tensor([rng.randrange(0, 30000)] * n, dtype=torch.int32, device="cuda")
            work_h = kv_ops.KVWorkList(
                torch.tensor([host.data_ptr() + i * geo.slot_size for i in range(n)], dtype=torch.int64, device="cuda"),
                blocks, deltas)
            work_d = kv_ops.KVWorkList(work_s.slot_ptrs, blocks, deltas)
            # end to end: file -> pinned host (O_DIRECT) -> fused kernel reading host memory -> pools
            lat = []
            for _ in range(5):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                eng.wait(eng.submit_read(host.data_ptr(), 0, nbytes))
                t1 = time.perf_counter()
                kv_ops.kv_restore(work_h, geo, pool, cos_sin, status)
                torch.cuda.synchronize()
                lat.append(((time.perf_counter() - t0) * 1e3, (t1 - t0) * 1e3))
            lat.sort()
            e2e_ms, read_ms = lat[len(lat) // 2]
            scat_ms, _ = time_cuda(lambda: kv_ops.kv_restore(work_d, geo, pool, cos_sin, status), iters=10)
            assert status.tolist() == [0, 0]
            out_bytes = nbytes  # fp8 pool: as many bytes written as read
            remote = out_bytes * (tp - 1) / tp if world > 1 else 0.0
            roof_ms = max((nbytes + out_bytes - remote) / hbm / 1e6, remote / NVLINK_GBS / 1e6)
            emit({"bench": "restore_sweep", "tokens": tokens, "slots": n, "MB": nbytes / 1e6, "gpus": world,
                  "tp": tp, "peers": "real" if world > 1 else "emulated on one GPU",
                  "io_backend": xfer.backend.name, "file_write_GBps": nbytes / w_s / 1e9,
                  "file_read_GBps": nbytes / (read_ms / 1e3) / 1e9, "save_kernel_ms": save_ms,
                  "scatter_ms": scat_ms, "scatter_GBps": (nbytes + out_bytes) / scat_ms / 1e6,
                  "scatter_frac_of_roofline": roof_ms / scat_ms, "roofline": f"{kind} HBM {hbm:.0f} GB/s, NVLink {NVLINK_GBS:.0f} GB/s",
                  "e2e_restore_ms": e2e_ms, "e2e_GBps": nbytes / e2e_ms / 1e6})
        if ctx is not None:
            dist.barrier(device_ids=[local])
    if rank == 0:
        xfer.close()
        os.unlink(path)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
