"""Shared-memory mailboxes between the ranks of one box (host side only: runs anywhere)."""

import multiprocessing as mp
import os
import time

import pytest

from daser_b200.parallel.mailbox import HostMailbox, MailboxTimeout


def _peer(path, rank, world, n, out):
    box = HostMailbox(path, rank, world)
    got = []
    for i in range(n):
        got.append(box.broadcast(None, src=0, timeout_s=20))
        everyone = box.gather({"rank": rank, "i": i}, timeout_s=20)
        assert [e["rank"] for e in everyone] == list(range(world)) and all(e["i"] == i for e in everyone)
    out.put((rank, got))
    box.close()


def test_broadcast_and_gather_between_processes(tmp_path):
    path = str(tmp_path / "mb")
    world, n = 3, 200
    lead = HostMailbox(path, 0, world, create=True)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_peer, args=(path, r, world, n, out)) for r in (1, 2)]
    for p in procs:
        p.start()
    try:
        for i in range(n):
            lead.broadcast({"step": i, "blocks": list(range(i % 7))})
            lead.gather({"rank": 0, "i": i}, timeout_s=20)
        results = dict(out.get(timeout=30) for _ in procs)
    finally:
        for p in procs:
            p.join(30)
        lead.close()
    for r in (1, 2):
        assert [m["step"] for m in results[r]] == list(range(n))
    assert not os.path.exists(path)


def test_timeout_overrun_and_latency(tmp_path):
    path = str(tmp_path / "mb")
    a = HostMailbox(path, 0, 2, create=True)
    b = HostMailbox(path, 1, 2)
    with pytest.raises(MailboxTimeout):
        b.receive(0, timeout_s=0.05)
    calls = []
    with pytest.raises(MailboxTimeout):
        b.receive(0, timeout_s=0.05, on_wait=lambda: calls.append(1))
    assert calls
    t0 = time.perf_counter()
    for i in range(100):
        a.publish(("plan", i, [0] * 64))
        assert b.receive(0)[1] == i
    assert (time.perf_counter() - t0) / 100 < 1e-3  # microseconds in practice
    for i in range(HostMailbox.RING + 1):  # the writer laps the reader
        a.publish(i)
    with pytest.raises(RuntimeError, match="overrun"):
        b.receive(0, timeout_s=0.05)
    with pytest.raises(ValueError):
        a.publish(b"x" * (a.slot_bytes + 1))
    b.close()
    a.close()
