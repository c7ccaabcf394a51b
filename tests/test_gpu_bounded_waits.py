"""Device-side waits run out instead of hanging: a flag that nothing sets makes the kernel return
with the status word set, and the stream and context stay usable.  (Nothing here faults, traps
or spins without a bound: the budget is two seconds of %globaltimer.)"""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_gemm_gate_timeout_sets_status_and_returns():
    from daser_b200.ops import gemm

    x = torch.ones(64, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(128, 128, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(1, dtype=torch.int32, device="cuda")  # nobody will ever set it
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    gemm.linear(x, w, gate_flags=flags.data_ptr(), gate_target=1, gate_rows=128, status=status)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert status.item() == 1
    assert 1.0 < waited < 20.0
    # the context is intact: the same GEMM with the flag set gives the right answer
    status.zero_()
    flags.fill_(1)
    out = gemm.linear(x, w, gate_flags=flags.data_ptr(), gate_target=1, gate_rows=128, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.all(out.float() == 128.0)


def test_norm_arrival_timeout_and_flag_wait_timeout():
    from daser_b200.ops import elementwise as ew

    x = torch.ones(4, 256, dtype=torch.bfloat16, device="cuda")
    wgt = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sync = ew.TpSync()
    sync.wait_counter, sync.wait_target = counter.data_ptr(), 5  # arrivals that never come
    sync.done_counter, sync.done_target = done.data_ptr(), 4
    sync.n_signal, sync.status = 0, status.data_ptr()
    out = ew.add_rmsnorm(x, wgt, tp_sync=sync)
    torch.cuda.synchronize()
    assert status.item() == 1 and done.item() == 4  # it still ran to the end so peers are not left waiting
    assert torch.isfinite(out.float()).all()
    status.zero_()
    ew.wait_flags(counter.data_ptr(), 1, 3, status)
    torch.cuda.synchronize()
    assert status.item() == 1
    status.zero_()
    counter.fill_(3)
    ew.wait_flags(counter.data_ptr(), 1, 3, status)
    torch.cuda.synchronize()
    assert status.item() == 0
