"""tcgen05 GEMM against an fp32 matmul of the same bf16 inputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, w):
    return x.float() @ w.float().t()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 512), (64, 1280, 8192), (1, 384, 256),
                                   (200, 136, 1000 * 8), (300, 512, 192)])
@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_store_epilogue(M, N, K, bn):
    from daser_b200.ops import gemm

    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = gemm.linear(x, w, block_n=bn, k_splits=1, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(x, w)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("M,N,K,ks", [(64, 1280, 8192, 8), (128, 256, 1024, 3), (5, 128, 4096, 16), (130, 320, 640, 2)])
def test_splitk_reduce_epilogue(M, N, K, ks):
    from daser_b200.ops import gemm

    torch.manual_seed(1)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    gemm.linear(x, w, acc=acc, k_splits=ks)
    torch.cuda.synchronize()
    ref = _ref(x, w)
    assert (acc - ref).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-3
    # accumulates: a second launch doubles it
    gemm.linear(x, w, acc=acc, k_splits=ks)
    torch.cuda.synchronize()
    assert (acc - 2 * ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 2e-3


def test_reduce_scatter_epilogue_emulated_ranks():
    """Two 'ranks' (K shards) on one device reduce into per-owner row buffers and bump the counters."""
    from daser_b200.ops import gemm

    torch.manual_seed(2)
    M, N, K, tp = 96, 256, 1024, 2
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    rows = M // tp
    bufs = [torch.zeros(rows, N, dtype=torch.float32, device="cuda") for _ in range(tp)]
    counters = torch.zeros(tp, dtype=torch.int32, device="cuda")
    for r in range(tp):
        ks = slice(r * K // tp, (r + 1) * K // tp)
        gemm.linear(x[:, ks], w[:, ks], owners=[b.data_ptr() for b in bufs], rows_per_owner=rows,
                    arrive=[counters.data_ptr() + 4 * i for i in range(tp)], ldc=N, block_n=128, k_splits=2)
    torch.cuda.synchronize()
    ref = _ref(x, w)
    got = torch.cat(bufs)
    assert (got - ref).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-3
    per_rank = gemm.expected_arrivals(M, N, 128, 2, rows, tp, K // tp)
    assert counters.tolist() == [c * tp for c in per_rank]


def test_gate_flags_release_the_loads():
    from daser_b200.ops import gemm

    torch.manual_seed(3)
    M, N, K = 256, 128, 256
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    flags = torch.full((2,), 5, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = gemm.linear(x, w, gate_flags=flags.data_ptr(), gate_target=5, gate_rows=128, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(x, w)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_bf16_scatter_epilogue_and_partial_sum_norm():
    """Reduce-scatter in its bf16 form, two 'ranks' on one device: each K shard stores its partial
    rows into its slot of the owners' receive buffers; the norm kernel sums the slots."""
    from daser_b200.ops import elementwise as ew
    from daser_b200.ops import gemm

    torch.manual_seed(4)
    M, N, K, tp = 48, 512, 1024, 2
    rows = M // tp
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    recv = [torch.zeros(tp * rows, N, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]  # per owner
    counters = torch.zeros(tp, dtype=torch.int32, device="cuda")
    for r in range(tp):
        ks = slice(r * K // tp, (r + 1) * K // tp)
        gemm.linear(x[:, ks], w[:, ks], owners=[b.data_ptr() for b in recv], rows_per_owner=rows, ldc=N,
                    scatter_bf16=True, dst_row_offset=r * rows, block_n=64,
                    arrive=[counters.data_ptr() + 4 * i for i in range(tp)])
    torch.cuda.synchronize()
    ref = x.float() @ w.float().t()
    per_rank = gemm.expected_arrivals(M, N, 64, 1, rows, tp, K // tp)
    assert counters.tolist() == [c * tp for c in per_rank]
    nw = torch.ones(N, dtype=torch.bfloat16, device="cuda")
    for owner in range(tp):
        summed = recv[owner].view(tp, rows, N).float().sum(0)
        want = ref[owner * rows : (owner + 1) * rows]
        assert (summed - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 2e-2
        res = torch.zeros(rows, N, dtype=torch.bfloat16, device="cuda")
        out = ew.add_rmsnorm(recv[owner][:rows], nw, residual=res, n_partials=tp, partial_stride=rows * N)
        torch.cuda.synchronize()
        h = summed.to(torch.bfloat16).float()
        assert torch.allclose(res.float(), h, atol=2e-2, rtol=2e-2)
        assert torch.allclose(out.float(), h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,N,K,ks", [(48, 512, 2048, 4), (130, 320, 1024, 3), (64, 8192, 4096, 4)])
def test_splitk_scatter_epilogue(M, N, K, ks):
    """Split-K partials meet in a local fp32 buffer; the last CTA of each tile scatters the bf16 sum
    into the owners' slots, zeroes the buffer and its tile counter, and bumps the arrival counters."""
    from daser_b200.ops import gemm

    torch.manual_seed(5)
    tp = 2
    rows = -(-M // tp)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    recv = [torch.zeros(tp * rows, N, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
    work = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    tiles = torch.zeros(1024, dtype=torch.int32, device="cuda")
    counters = torch.zeros(tp, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):  # the second launch must find the work buffer and counters clean
        gemm.linear(x, w, owners=[b.data_ptr() for b in recv], rows_per_owner=rows, ldc=N, scatter_bf16=True,
                    dst_row_offset=1 * rows, block_n=128, k_splits=ks, work=work, tile_counters=tiles,
                    arrive=[counters.data_ptr() + 4 * i for i in range(tp)], status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert work.abs().max().item() == 0 and tiles.abs().max().item() == 0
    ref = x.float() @ w.float().t()
    for owner in range(tp):
        n = min(rows, M - owner * rows)
        got = recv[owner].view(tp, rows, N)[1, :n].float()  # slot 1 = this "rank"
        want = ref[owner * rows : owner * rows + n]
        assert (got - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-2
        assert recv[owner].view(tp, rows, N)[0].abs().max().item() == 0
    per = gemm.expected_arrivals(M, N, 128, 1, rows, tp, K)
    assert counters.tolist() == [2 * c for c in per]


@pytest.mark.parametrize("ks", [1, 4])
def test_broadcast_epilogue_is_a_one_shot_all_reduce(ks):
    """Two 'ranks' on one device: each K shard stores its whole bf16 partial into its slot of BOTH
    receive buffers and bumps both arrival counters once per tile; every buffer then sums to x w^T."""
    from daser_b200.ops import elementwise as ew
    from daser_b200.ops import gemm

    torch.manual_seed(6)
    M, N, K, tp, cap = 40, 512, 4096, 2, 64
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    recv = [torch.zeros(tp * cap, N, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
    counters = torch.zeros(tp, dtype=torch.int32, device="cuda")
    work = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    tiles = torch.zeros(256, dtype=torch.int32, device="cuda")
    bn = 128 if ks > 1 else 64
    for r in range(tp):
        sl = slice(r * K // tp, (r + 1) * K // tp)
        gemm.linear(x[:, sl], w[:, sl], owners=[b.data_ptr() for b in recv], rows_per_owner=cap, ldc=N,
                    scatter_bf16=True, dst_row_offset=r * cap, block_n=bn, k_splits=ks, broadcast=True,
                    work=work, tile_counters=tiles, arrive=[counters.data_ptr() + 4 * i for i in range(tp)])
    torch.cuda.synchronize()
    assert counters.tolist() == [tp * (N // bn)] * tp
    assert work.abs().max().item() == 0 and tiles.abs().max().item() == 0
    ref = x.float() @ w.float().t()
    for dst in range(tp):
        summed = recv[dst].view(tp, cap, N)[:, :M].float().sum(0)
        assert (summed - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2
        assert recv[dst].view(tp, cap, N)[:, M:].abs().max().item() == 0  # rows past M untouched
    res = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    out = ew.add_rmsnorm(recv[1][:M], torch.ones(N, dtype=torch.bfloat16, device="cuda"), residual=res,
                         n_partials=tp, partial_stride=cap * N)
    torch.cuda.synchronize()
    h = recv[1].view(tp, cap, N)[:, :M].float().sum(0).to(torch.bfloat16).float()
    assert torch.allclose(out.float(), h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,inter,K", [(64, 512, 1024), (33, 1024, 256), (130, 19456, 512)])
def test_swiglu_epilogue_matches_gemm_then_activation(M, inter, K):
    """Gate/up rows interleaved in blocks of 64: the GEMM's epilogue applies silu(gate) * up."""
    from daser_b200.ops import elementwise as ew
    from daser_b200.ops import gemm

    torch.manual_seed(7)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, device="cuda") * 0.1).to(torch.bfloat16)  # [gate | up]
    w_il = gemm.interleave_gate_up(w)
    out = torch.full((M, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    gemm.linear_swiglu(x, w_il, out)
    torch.cuda.synchronize()
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2
    # the unfused pair on the interleaved layout gives the same thing
    gu_il = gemm.linear(x, w_il, out=torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda"), k_splits=1)
    y = ew.swiglu(gu_il, block=gemm.GATE_UP_BLOCK)
    torch.cuda.synchronize()
    assert (y.float() - ref).abs().max().item() <= 3e-2 * ref.abs().max().item() + 3e-2
