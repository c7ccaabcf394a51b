"""One small, self-terminating launch of a hot kernel, sized for an ``ncu`` capture.

    python benchmarks/profile_case.py --case restore|save|gemm|gemm_rs|gemm_qkv_rope|attn_decode|attn_prefill|rmsnorm

Each case touches a few hundred MB at most (larger than L2, far from the GPU's capacity),
runs two warm-up launches and three measured ones, and prints the CUDA-event time of the
last.  Captures of these cases end by themselves in about a minute under ``--set full``.
"""

from __future__ import annotations

import argparse

import torch

from _common import emit, time_cuda

from daser_b200.kv.layout import KVGeometry
from daser_b200.ops import attention, elementwise as ew, gemm, kv_ops
from daser_b200.position import inv_freq_table


def case_restore(save=False):
    geo = KVGeometry(80, 8, 128, 16, 2, "fp8b16")
    n = 32  # 32 slots = 512 tokens of Llama-3-70B KV = 105 MB of images
    staging = torch.randint(0, 120, (n * geo.slot_size,), dtype=torch.uint8, device="cuda")
    pay = [torch.zeros(80, n + 4, 2, 8, 16, 128, dtype=torch.uint8, device="cuda")]
    sc = [torch.ones(80, n + 4, 2, 8, 16, 8, dtype=torch.float32, device="cuda")]
    pool = kv_ops.PagedKVPool.from_tensors(pay, sc, "LNKHTD")
    work = kv_ops.KVWorkList(
        torch.tensor([staging.data_ptr() + i * geo.slot_size for i in range(n)], dtype=torch.int64, device="cuda"),
        torch.randperm(n + 4, device="cuda")[:n].to(torch.int32), torch.full((n,), 777, dtype=torch.int32, device="cuda"))
    cos_sin = kv_ops.rope_table(8192, inv_freq_table(128, 500000.0), "cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    if save:
        return (lambda: kv_ops.kv_save(work, geo, pool, 0, status)), 2 * n * geo.slot_size
    return (lambda: kv_ops.kv_restore(work, geo, pool, cos_sin, status)), 2 * n * geo.slot_size


def case_gemm(reduce_scatter=False):
    M, N, K = 64, 8192, 8192  # 134 MB of weights: streams from HBM
    x = (torch.randn(M, K, device="cuda") * 0.1).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    bn, ks = gemm.plan_tiles(M, N, K, True)
    if reduce_scatter:
        # two "ranks" emulated on one device: rows split over two owner buffers, arrival counters bumped
        bufs = [torch.zeros(32, N, dtype=torch.float32, device="cuda") for _ in range(2)]
        cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
        fn = lambda: gemm.linear(x, w, owners=[b.data_ptr() for b in bufs], rows_per_owner=32, ldc=N, block_n=bn,
                                 k_splits=ks, arrive=[cnt.data_ptr(), cnt.data_ptr() + 4])
    else:
        acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        fn = lambda: gemm.linear(x, w, acc=acc, block_n=bn, k_splits=ks)
    return fn, 2 * (N * K + M * K) + 4 * M * N


def case_gemm_qkv_rope():
    """The QKV projection of Llama-3-70B for a 64-token step with RoPE + fp8 quantise + the paged KV
    write as its epilogue (opt-in in the engine: `DASER_FUSE_QKV_ROPE=1`); 168 MB of weights."""
    T, K, Hq, Hkv, D, B = 64, 8192, 64, 8, 128, 16
    N = (Hq + 2 * Hkv) * D
    x = (torch.randn(T, K, device="cuda") * 0.1).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    n_blocks = T // B + 4
    positions = (torch.arange(T, device="cuda") + 3328).to(torch.int32)
    slot_mapping = (torch.randperm(n_blocks, device="cuda")[torch.arange(T, device="cuda") // B] * B
                    + torch.arange(T, device="cuda") % B).to(torch.int64)
    cos_sin = kv_ops.rope_table(8192, inv_freq_table(D, 500000.0), "cuda")
    pay = torch.zeros(1, n_blocks, 2, Hkv, B, D, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(1, n_blocks, 2, Hkv, B, D // 16, dtype=torch.float32, device="cuda")
    pool = kv_ops.PagedKVPool.from_tensors([pay], [sc], "LNKHTD")
    work = torch.zeros(T, N, dtype=torch.float32, device="cuda")
    counters = torch.zeros(256, dtype=torch.int32, device="cuda")
    q_out = torch.zeros(T, Hq, D, dtype=torch.bfloat16, device="cuda")
    _, ks = gemm.plan_tiles(T, N, K, True)
    fn = lambda: gemm.linear_qkv_rope(x, w, positions, slot_mapping, cos_sin, q_out, Hq, Hkv, B, pool, 0, 0, work,
                                      counters, k_splits=ks)
    return fn, 2 * (N * K + T * K) + 2 * T * Hq * D


def case_attn(prefill=False):
    Hq, Hkv, D, B = 64, 8, 128, 16
    batch, ctx = (1, 4096) if prefill else (16, 8192)
    qlen = 64 if prefill else 1
    nb = batch * ctx // B
    payload = torch.randint(0, 120, (1, nb, 2, Hkv, B, D), dtype=torch.uint8, device="cuda")
    scales = torch.full((1, nb, 2, Hkv, B, D // 16), 0.01, dtype=torch.float32, device="cuda")
    pool = kv_ops.PagedKVPool.from_tensors([payload], [scales], "LNKHTD")
    tables = torch.randperm(nb, device="cuda").to(torch.int32).view(batch, ctx // B)
    q = torch.randn(batch * qlen, Hq, D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    q_start = (torch.arange(batch + 1, device="cuda") * qlen).to(torch.int32)
    ctx_t = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    ws = attention.AttentionWorkspace("cuda")
    ns, st = attention.plan_splits(batch, Hkv, qlen, Hq // Hkv, ctx, B)
    fn = lambda: attention.paged_attention(q, out, pool, 0, tables, q_start, ctx_t, qlen, ctx, Hkv, D**-0.5, ws,
                                           nsplit=ns, split_tokens=st)
    return fn, batch * ctx * 2 * Hkv * D * 1.25


def case_rmsnorm():
    T, H = 4096, 8192
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    o = torch.empty_like(x)
    return (lambda: ew.add_rmsnorm(x, w, residual=res, out=o)), T * H * 2 * 4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    args = ap.parse_args()
    table = {
        "restore": lambda: case_restore(False), "save": lambda: case_restore(True),
        "gemm": lambda: case_gemm(False), "gemm_rs": lambda: case_gemm(True), "gemm_qkv_rope": case_gemm_qkv_rope,
        "attn_decode": lambda: case_attn(False), "attn_prefill": lambda: case_attn(True),
        "rmsnorm": case_rmsnorm,
    }
    fn, nbytes = table[args.case]()
    med, best = time_cuda(fn, iters=3, warmup=2, flush=True)
    emit({"case": args.case, "ms": med, "best_ms": best, "algorithmic_GB": nbytes / 1e9, "GBps": nbytes / med / 1e6})


if __name__ == "__main__":
    main()
