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


def test_tp_pick_token_with_the_peers_arrival_posted_and_with_it_missing():
    """The sampling exchange as rank 0 of 2 on one GPU: the peer's candidates and arrival are
    written by hand before the launch (two kernels that wait for each other never share a GPU).
    Two rounds, so that both halves of the table and the replay through `epoch` are used; then a
    round in which the peer never arrives: the wait runs out, the status word says so."""
    from daser_b200.ops import elementwise as ew

    tp, cap, n = 2, 64, 5
    mine = torch.zeros(2 * tp * 2 * cap, dtype=torch.float32, device="cuda")   # rank 0's table
    theirs = torch.zeros_like(mine)                                           # stands in for rank 1's table
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")                # [0]: rank 0's, [1]: rank 1's
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(n, dtype=torch.int32, device="cuda")
    view = mine.view(2, tp, 2, cap)
    for rnd in range(2):
        my_val = torch.tensor([1.0, 5.0, -2.0, 0.5, 3.0], device="cuda") + rnd
        my_idx = torch.tensor([10, 11, 12, 13, 14], dtype=torch.int32, device="cuda")
        peer_val = torch.tensor([2.0, 4.0, -1.0, 0.5, 9.0], device="cuda")
        peer_idx = torch.tensor([110, 111, 112, 113, 114], dtype=torch.int32, device="cuda")
        view[rnd, 1, 0, :n] = peer_val                       # what rank 1's kernel would have stored here
        view[rnd, 1, 1, :n] = peer_idx.view(torch.float32)
        counters[0] += 1                                     # ... and its arrival
        ew.tp_pick_token(my_val, my_idx, n, 0, tp, cap, [mine.data_ptr(), theirs.data_ptr()],
                         [counters[0:].data_ptr(), counters[1:].data_ptr()], epoch, status, out)
        torch.cuda.synchronize()
        want = torch.where(my_val >= peer_val, my_idx, peer_idx)  # ties go to the lower rank
        assert status.item() == 0 and out.tolist() == want.tolist()
        assert epoch.item() == tp * (rnd + 1) and counters.tolist() == [tp * (rnd + 1), rnd + 1]
        # this rank's candidates reached the peer's table, in the round's half
        assert theirs.view(2, tp, 2, cap)[rnd, 0, 0, :n].tolist() == my_val.tolist()
    ew.tp_pick_token(my_val, my_idx, n, 0, tp, cap, [mine.data_ptr(), theirs.data_ptr()],
                     [counters[0:].data_ptr(), counters[1:].data_ptr()], epoch, status, out)
    torch.cuda.synchronize()
    assert status.item() == 1
