"""The native lookup thread: same answers as the Python server, at every point of a chunk's life."""

import os
import random
import socket
import struct

import msgpack
import pytest

from conftest import LiveControlPlane
from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.server.native_index import FastLookupServer

pytestmark = pytest.mark.skipif(not FastLookupServer.supported(), reason="native library not built")


def _pair(lp):
    """(client on the main socket only, client that negotiated the native socket)"""
    plain, fast = IPCClientSync(lp.socket_path), IPCClientSync(lp.socket_path)
    fast.negotiate()
    assert fast._fast is not None and plain._fast is None
    return plain, fast


def test_native_socket_agrees_with_the_python_server_through_a_ring_lifetime(tmp_path):
    lp = LiveControlPlane(tmp_path, total_slots=24).start()     # small ring: allocations evict
    plain, fast = _pair(lp)
    rng = random.Random(0)
    keys = [f"{rng.getrandbits(128):032x}" for _ in range(40)] + ["not-a-digest", "clé-ünïcode"]
    reserved, committed = [], []
    try:
        for step in range(300):
            op = rng.random()
            if op < 0.4:
                key = rng.choice(keys)
                try:
                    plain.alloc_chunk(key, 16 * rng.randint(1, 3), rng.choice(["m", "m", "other"]))
                    reserved.append(key)
                except RuntimeError:
                    pass                                           # already stored under another size
            elif op < 0.7 and reserved:
                key = reserved.pop(rng.randrange(len(reserved)))
                try:
                    plain.commit_chunk(key)
                    committed.append(key)
                except RuntimeError:
                    pass                                           # evicted before the commit
            elif op < 0.8 and committed:
                plain.evict_chunk(committed.pop(rng.randrange(len(committed))))
            elif op < 0.85 and reserved:
                plain.abort_chunk(reserved.pop(rng.randrange(len(reserved))))
            probe = rng.sample(keys, 6)
            for model in ("m", "other"):
                assert fast.lookup_chunks(probe, model) == plain.lookup_chunks(probe, model), f"step {step}"
        assert any(c is not None for c in fast.lookup_chunks(keys, "m"))
        stats = plain.stats()["fast_lookup"]
        assert stats["calls"] >= 600 and stats["hits"] > 0 and stats["misses"] > 0
    finally:
        plain.close()
        fast.close()
        lp.stop()


def test_commit_is_visible_on_the_native_socket_when_it_is_acknowledged_and_parts_are_respected(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    plain, fast = _pair(lp)
    try:
        plain.alloc_chunk("a" * 32, 32, "m")
        assert fast.lookup_chunks(["a" * 32], "m") == [None]           # reserved, not visible
        plain.commit_chunk("a" * 32, part=0, parts=2)
        assert fast.lookup_chunks(["a" * 32], "m") == [None]           # one part of two
        plain.commit_chunk("a" * 32, part=1, parts=2)
        got = fast.lookup_chunks(["a" * 32], "m")[0]
        assert got == plain.lookup_chunks(["a" * 32], "m")[0] and got["file_offset"] == got["start_slot"] * 4096
    finally:
        plain.close()
        fast.close()
        lp.stop()


def test_snapshot_restart_refills_the_native_table_and_clients_fall_back_when_it_is_gone(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    c = IPCClientSync(lp.socket_path)
    c.alloc_chunk("b" * 32, 16, "m")
    c.commit_chunk("b" * 32)
    c.alloc_chunk("c" * 32, 16, "m")                                   # reserved only
    c.close()
    lp.stop(save=True)
    lp2 = LiveControlPlane(tmp_path).start()
    plain, fast = _pair(lp2)
    try:
        assert fast.lookup_chunks(["b" * 32, "c" * 32], "m") == plain.lookup_chunks(["b" * 32, "c" * 32], "m")
        assert fast.lookup_chunks(["b" * 32], "m")[0] is not None
        # the native thread goes away (here: stopped by hand); the client keeps working on the main socket
        lp2.plane.server._fast.stop()
        assert fast.lookup_chunks(["b" * 32], "m") == plain.lookup_chunks(["b" * 32], "m")
        assert fast._fast is None
    finally:
        plain.close()
        fast.close()
        lp2.stop()
    assert not os.path.exists(lp2.socket_path + ".fast")


def test_other_operations_and_bad_frames_on_the_native_socket(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    path = lp.socket_path + ".fast"

    def call(sock, obj):
        body = msgpack.packb(obj)
        sock.sendall(struct.pack(">I", len(body)) + body)
        n = struct.unpack(">I", sock.recv(4, socket.MSG_WAITALL))[0]
        return msgpack.unpackb(sock.recv(n, socket.MSG_WAITALL))

    try:
        s = socket.socket(socket.AF_UNIX)
        s.connect(path)
        assert "error" in call(s, {"op": "alloc_chunk", "chunk_key": "x", "token_count": 16})
        assert "error" in call(s, {"op": "lookup_chunks", "tokens": [1, 2, 3], "model_id": "m"})
        assert "error" in call(s, [1, 2, 3])
        # unknown fields of any type are skipped; two requests in one write are both answered
        extra = {"op": "lookup_chunks", "keys": ["k"], "model_id": "m", "x": {"a": [1, -2.5, None, True, b"bin", 2**40]}}
        assert call(s, extra) == {"chunks": [None]}
        body = msgpack.packb({"op": "lookup_chunks", "keys": [], "model_id": "m"})
        s.sendall((struct.pack(">I", len(body)) + body) * 2)
        for _ in range(2):
            n = struct.unpack(">I", s.recv(4, socket.MSG_WAITALL))[0]
            assert msgpack.unpackb(s.recv(n, socket.MSG_WAITALL)) == {"chunks": []}
        # a frame that claims 4 GiB, and a truncated map: the connection is closed, nothing else
        s.sendall(b"\xff\xff\xff\xff")
        assert s.recv(1) == b""
        s.close()
        s = socket.socket(socket.AF_UNIX)
        s.connect(path)
        assert call(s, {"op": "lookup_chunks", "keys": ["k"]}) == {"chunks": [None]}   # model_id defaults
        s.sendall(struct.pack(">I", 3) + b"\x82\xa2o")
        n = struct.unpack(">I", s.recv(4, socket.MSG_WAITALL))[0]
        assert "error" in msgpack.unpackb(s.recv(n, socket.MSG_WAITALL))
        s.close()
        c = IPCClientSync(lp.socket_path)
        c.negotiate()
        assert c.lookup_chunks(["k"], "m") == [None]                  # the thread is still serving
        c.close()
    finally:
        lp.stop()


def test_wide_requests_cover_the_longer_msgpack_forms(tmp_path):
    """More than 15 keys (array16), keys longer than 31 bytes (str8) and than 255 (str16), slots
    beyond 32 bits of file offset: the native encoder and decoder against msgpack's own."""
    lp = LiveControlPlane(tmp_path, total_slots=64, slot_size=1 << 28).start()     # 256 MiB slots: offsets > 4 GiB
    plain, fast = _pair(lp)
    try:
        keys = [f"key-{i:03d}-" + "x" * (10 + 9 * i) for i in range(40)]          # 17 .. 368 characters
        for i, k in enumerate(keys[:30]):
            plain.alloc_chunk(k, 16, "m")
            plain.commit_chunk(k)
        got = fast.lookup_chunks(keys, "m")
        assert got == plain.lookup_chunks(keys, "m")
        assert sum(g is not None for g in got) == 30 and got[29]["file_offset"] == 29 * (1 << 28) > 2**32
        assert fast.lookup_chunks([], "m") == []
    finally:
        plain.close()
        fast.close()
        lp.stop()


def test_negotiation_is_retried_until_a_server_answers(tmp_path):
    """A scheduler half that comes up before the control plane must not settle for the slow path."""
    from daser_b200.connector.core import SchedulerHalf

    sock = str(tmp_path / "d.sock")
    half = SchedulerHalf(sock, 16, "m")
    assert half.plan_chunk_loads("r0", [("k" * 32, 0)]) == [None]         # nobody there: a miss, and not negotiated
    assert half._negotiated is False
    lp = LiveControlPlane(tmp_path).start()
    try:
        assert half.plan_chunk_loads("r1", [("k" * 32, 0)]) == [None]
        assert half._negotiated is True and half._ipc._fast is not None and half._ipc.binary_tokens
    finally:
        half.close()
        lp.stop()
