"""Failures injected on the host: transport, frames, restart, snapshot corruption."""

import socket
import struct

import msgpack
import pytest

from conftest import LiveControlPlane
from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.hashing import hash_tokens
from daser_b200.proto import frames


def test_client_reconnects_after_server_restart(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    c = IPCClientSync(lp.socket_path, timeout=5)
    assert c.lookup([1] * 16, "m") == []
    lp.stop(save=True)
    lp2 = LiveControlPlane(tmp_path).start()
    try:
        assert c.lookup([1] * 16, "m") == []  # one transparent retry
    finally:
        lp2.stop()
        c.close()


def test_client_raises_runtimeerror_when_server_is_gone(tmp_path):
    c = IPCClientSync(str(tmp_path / "absent.sock"), timeout=1)
    with pytest.raises(RuntimeError, match="failed"):
        c.lookup([1], "m")


def test_oversized_and_truncated_frames_do_not_kill_the_server(live_plane):
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.connect(live_plane.socket_path)
    s.sendall(struct.pack(">I", frames.MAX_FRAME + 1))
    s.settimeout(5)
    data = s.recv(1 << 16)
    assert b"exceeds limit" in data
    s.close()
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.connect(live_plane.socket_path)
    s.sendall(struct.pack(">I", 100) + b"abc")  # then hang up mid-frame
    s.close()
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.connect(live_plane.socket_path)
    s.sendall(struct.pack(">I", 3) + b"\xc1\xc1\xc1")  # invalid msgpack
    s.settimeout(5)
    assert b"error" in s.recv(1 << 16)
    s.close()
    c = IPCClientSync(live_plane.socket_path)
    assert c.lookup([1] * 16, "m") == []
    c.close()


def test_torn_write_stays_invisible_across_restart(tmp_path):
    """Crash between the data write and the commit: the chunk must not come back."""
    lp = LiveControlPlane(tmp_path).start()
    c = IPCClientSync(lp.socket_path)
    done, torn = list(range(32)), list(range(100, 132))
    c.alloc_chunk(hash_tokens(done), 32, "default")
    c.commit_chunk(hash_tokens(done))
    c.alloc_chunk(hash_tokens(torn), 32, "default")  # never committed
    c.close()
    lp.stop(save=True)
    lp2 = LiveControlPlane(tmp_path).start()
    try:
        c = IPCClientSync(lp2.socket_path)
        assert len(c.lookup(done, "default")) == 1
        assert c.lookup(torn, "default") == []
        assert c.lookup_chunks([hash_tokens(torn)], "default") == [None]
        # and its slots were released for reuse
        assert c.stats()["ring"]["used_slots"] == 2
        c.close()
    finally:
        lp2.stop()


def test_corrupt_snapshot_means_cold_start(tmp_path):
    (tmp_path / "daser.index").write_bytes(b"\x00garbage\xff" * 10)
    lp = LiveControlPlane(tmp_path).start()
    try:
        c = IPCClientSync(lp.socket_path)
        assert c.stats()["ring"]["chunks"] == 0
        c.close()
    finally:
        lp.stop()


def test_snapshot_write_is_atomic(tmp_path, monkeypatch):
    """A failure while writing leaves the previous snapshot intact."""
    import os

    from daser_b200.server import metadata_store as ms

    path = str(tmp_path / "snap")
    ms.atomic_write(path, b"old")
    real_replace = os.replace

    def boom(*a, **k):
        raise OSError("disk went away")

    monkeypatch.setattr(os, "replace", boom)
    with pytest.raises(OSError):
        ms.atomic_write(path, b"new-new-new")
    monkeypatch.setattr(os, "replace", real_replace)
    assert open(path, "rb").read() == b"old"


def test_periodic_snapshot(tmp_path):
    import time

    lp = LiveControlPlane(tmp_path, snapshot_interval_s=0.05).start()
    try:
        c = IPCClientSync(lp.socket_path)
        c.alloc_chunk("k", 16, "default")
        c.commit_chunk("k")
        deadline = time.time() + 5
        while not (tmp_path / "daser.index").exists() and time.time() < deadline:
            time.sleep(0.02)
        raw = msgpack.unpackb((tmp_path / "daser.index").read_bytes(), raw=False)
        assert set(raw) >= {"head", "tail", "index", "doc_registry"}
        c.close()
    finally:
        lp.stop()


def test_worker_refuses_a_control_plane_with_another_geometry(tmp_path):
    import torch

    from daser_b200.connector.core import TorchKVBackend, WorkerHalf
    from daser_b200.kv.layout import KVGeometry

    geo = KVGeometry(2, 2, 32, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, slot_size=geo.slot_size * 2).start()  # server configured for other slots
    try:
        pool = torch.zeros(2, 8, 2, 2, 16, 32)
        with pytest.raises(ValueError, match="disagree"):
            WorkerHalf(lp.socket_path, lp.cfg.store_path, geo, TorchKVBackend(geo, pool, [1.0] * 16))
    finally:
        lp.stop()


def test_offset_scan_finds_chunks_again_after_a_restart(tmp_path):
    """The first-block anchors that the offset scan needs are part of the snapshot: a chunk
    committed before a restart is still found inside a prompt after it."""
    lp = LiveControlPlane(tmp_path).start()
    c = IPCClientSync(lp.socket_path)
    chunk = list(range(300, 332))
    key = hash_tokens(chunk)
    c.alloc_chunk(key, 32, "default")
    c.commit_chunk(key, first_block=hash_tokens(chunk[:16]))
    prompt = [9] * 16 + chunk + [4, 5]
    before = c.scan_chunks(prompt, "default")
    assert [(h["chunk_key"], h["offset"]) for h in before] == [(key, 16)]
    c.close()
    lp.stop(save=True)
    lp2 = LiveControlPlane(tmp_path).start()
    try:
        c = IPCClientSync(lp2.socket_path)
        after = c.scan_chunks(prompt, "default")
        assert [(h["chunk_key"], h["offset"]) for h in after] == [(key, 16)]
        c.close()
    finally:
        lp2.stop()
