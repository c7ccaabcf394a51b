"""Component tests over a real Unix socket with hand-packed frames."""

import socket
import struct

import msgpack
import pytest

from daser_b200.connector.ipc_client import IPCClientAsync, IPCClientSync
from daser_b200.hashing import hash_tokens


def rpc(path, payload, sock=None):
    own = sock is None
    s = sock or socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    if own:
        s.connect(path)
    body = msgpack.packb(payload, use_bin_type=True)
    s.sendall(struct.pack(">I", len(body)) + body)
    hdr = b""
    while len(hdr) < 4:
        hdr += s.recv(4 - len(hdr))
    (n,) = struct.unpack(">I", hdr)
    buf = b""
    while len(buf) < n:
        buf += s.recv(n - len(buf))
    if own:
        s.close()
    return msgpack.unpackb(buf, raw=False)


def test_alloc_offsets(live_plane):
    p = live_plane.socket_path
    r1 = rpc(p, {"op": "alloc_chunk", "chunk_key": "a", "token_count": 33, "model_id": "m"})
    assert r1 == {"start_slot": 0, "num_slots": 3, "file_offset": 0, "pos_offset": 0}
    r2 = rpc(p, {"op": "alloc_chunk", "chunk_key": "b", "token_count": 16, "model_id": "m"})
    assert r2["start_slot"] == 3 and r2["file_offset"] == 3 * 4096


def test_two_phase_visibility(live_plane):
    p = live_plane.socket_path
    toks = list(range(32))
    key = hash_tokens(toks)
    rpc(p, {"op": "alloc_chunk", "chunk_key": key, "token_count": 32, "model_id": "m"})
    assert rpc(p, {"op": "lookup", "tokens": toks, "model_id": "m"}) == {"chunks": []}
    assert rpc(p, {"op": "commit_chunk", "chunk_key": key}) == {"ok": True}
    got = rpc(p, {"op": "lookup", "tokens": toks + [5, 6, 7], "model_id": "m"})["chunks"]
    assert len(got) == 1
    assert set(got[0]) == {
        "chunk_key", "start_slot", "num_slots", "token_count", "pos_offset",
        "model_id", "file_offset",
    }
    assert got[0]["token_count"] == 32
    # model isolation
    assert rpc(p, {"op": "lookup", "tokens": toks, "model_id": "other"}) == {"chunks": []}


def test_match_and_alloc_miss_then_hit_and_idempotence(live_plane):
    p = live_plane.socket_path
    toks = list(range(40))  # 2 full blocks
    key = hash_tokens(toks[:32])
    req = {"op": "match_and_alloc", "tokens": toks, "chunk_key": key, "model_id": "m"}
    r = rpc(p, req)
    assert r["chunks"] == [] and r["alloc"]["token_count"] == 32
    assert r["alloc"]["num_slots"] == 2
    # the engine may ask again before the store finished: same reservation, no error
    assert rpc(p, req)["alloc"]["start_slot"] == r["alloc"]["start_slot"]
    rpc(p, {"op": "commit_chunk", "chunk_key": key})
    r = rpc(p, req)
    assert r["alloc"] is None and r["chunks"][0]["chunk_key"] == key
    # empty key or sub-block prompt: nothing reserved
    assert rpc(p, dict(req, tokens=[1, 2, 3], chunk_key="x"))["alloc"] is None
    assert rpc(p, dict(req, tokens=list(range(100, 140)), chunk_key=""))["alloc"] is None


def test_errors_keep_the_connection_alive(live_plane):
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.connect(live_plane.socket_path)
    assert rpc(None, {"op": "bogus"}, s) == {"error": "unknown op: bogus"}
    assert "error" in rpc(None, {"op": "commit_chunk", "chunk_key": "nope"}, s)
    assert "error" in rpc(None, {"op": "alloc_chunk"}, s)  # missing fields
    assert "chunks" in rpc(None, {"op": "lookup", "tokens": [1], "model_id": "m"}, s)
    s.close()


def test_evict_chunk_hides_it(live_plane):
    p = live_plane.socket_path
    toks = list(range(16))
    key = hash_tokens(toks)
    rpc(p, {"op": "alloc_chunk", "chunk_key": key, "token_count": 16, "model_id": "m"})
    rpc(p, {"op": "commit_chunk", "chunk_key": key})
    assert rpc(p, {"op": "evict_chunk", "chunk_key": key}) == {"ok": True}
    assert rpc(p, {"op": "lookup", "tokens": toks, "model_id": "m"}) == {"chunks": []}


def test_ring_eviction_invalidates_the_index(tmp_path):
    from conftest import LiveControlPlane

    lp = LiveControlPlane(tmp_path, total_slots=4).start()
    try:
        p = lp.socket_path
        keys = []
        for i in range(3):  # 3 x 2 slots into a 4-slot ring: the first is overwritten
            toks = list(range(i * 100, i * 100 + 32))
            keys.append((toks, hash_tokens(toks)))
            rpc(p, {"op": "alloc_chunk", "chunk_key": keys[-1][1], "token_count": 32, "model_id": "m"})
            rpc(p, {"op": "commit_chunk", "chunk_key": keys[-1][1]})
        assert rpc(p, {"op": "lookup", "tokens": keys[0][0], "model_id": "m"}) == {"chunks": []}
        assert len(rpc(p, {"op": "lookup", "tokens": keys[2][0], "model_id": "m"})["chunks"]) == 1
    finally:
        lp.stop()


def test_lookup_chunks_abort_hello_stats(live_plane):
    p = live_plane.socket_path
    toks = list(range(500, 548))
    key = hash_tokens(toks)
    rpc(p, {"op": "alloc_chunk", "chunk_key": key, "token_count": 48, "model_id": "m"})
    got = rpc(p, {"op": "lookup_chunks", "keys": [key, "zz"], "model_id": "m"})
    assert got["chunks"] == [None, None]  # reserved but not committed
    rpc(p, {"op": "commit_chunk", "chunk_key": key, "first_block": hash_tokens(toks[:16])})
    got = rpc(p, {"op": "lookup_chunks", "keys": [key, "zz"], "model_id": "m"})
    assert got["chunks"][0]["num_slots"] == 3 and got["chunks"][1] is None
    prompt = list(range(32)) + toks + [9] * 20
    hits = rpc(p, {"op": "lookup_chunks", "tokens": prompt, "model_id": "m"})["hits"]
    assert [(h["chunk_key"], h["offset"]) for h in hits] == [(key, 32)]
    rpc(p, {"op": "alloc_chunk", "chunk_key": "tmp", "token_count": 16, "model_id": "m"})
    assert rpc(p, {"op": "abort_chunk", "chunk_key": "tmp"})["released"] is True
    assert rpc(p, {"op": "abort_chunk", "chunk_key": key})["released"] is False
    assert rpc(p, {"op": "hello", "geometry": {"slot_size": 4096}})["ok"]
    assert "geometry mismatch" in rpc(p, {"op": "hello", "geometry": {"slot_size": 1}})["error"]
    assert rpc(p, {"op": "stats"})["ring"]["used_slots"] == 3


def test_doc_ops(live_plane):
    p = live_plane.socket_path
    keys = []
    for i in range(2):
        k = f"chunk{i}"
        keys.append(k)
        rpc(p, {"op": "alloc_chunk", "chunk_key": k, "token_count": 16, "model_id": "m"})
        rpc(p, {"op": "commit_chunk", "chunk_key": k})
    r = rpc(p, {"op": "register_doc", "doc_id": "d1", "title": "T", "chunk_keys": keys + ["gone"],
                "token_count": 48, "tokens": list(range(48))})
    assert r == {"ok": True, "chunk_count_cached": 2}
    assert "error" in rpc(p, {"op": "register_doc", "doc_id": "d1", "title": "T", "chunk_keys": []})
    docs = rpc(p, {"op": "list_docs"})["docs"]
    assert docs[0]["chunk_count_total"] == 3 and docs[0]["chunk_count_cached"] == 2
    assert set(docs[0]) == {"doc_id", "title", "token_count", "chunk_count_total",
                            "chunk_count_cached", "status", "created_at"}
    doc = rpc(p, {"op": "get_doc", "doc_id": "d1"})["doc"]
    assert doc["cached_mask"] == [True, True, False] and doc["tokens"] == list(range(48))
    assert "error" in rpc(p, {"op": "get_doc", "doc_id": "nope"})
    # evict_chunk cascades into the mask
    rpc(p, {"op": "evict_chunk", "chunk_key": "chunk0"})
    assert rpc(p, {"op": "get_doc", "doc_id": "d1"})["doc"]["cached_mask"] == [False, True, False]
    # a second doc shares chunk1: evicting d1 must keep it
    rpc(p, {"op": "register_doc", "doc_id": "d2", "title": "", "chunk_keys": ["chunk1"], "token_count": 16})
    assert rpc(p, {"op": "evict_doc", "doc_id": "d1"}) == {"ok": True, "chunks_evicted": 0}
    assert rpc(p, {"op": "evict_doc", "doc_id": "d2"}) == {"ok": True, "chunks_evicted": 1}
    assert "error" in rpc(p, {"op": "evict_doc", "doc_id": "d2"})


def test_sync_client(live_plane):
    c = IPCClientSync(live_plane.socket_path)
    toks = list(range(64))
    assert c.lookup(toks, "m") == []
    chunks, alloc = c.match_and_alloc(toks, hash_tokens(toks), "m")
    assert chunks == [] and alloc["num_slots"] == 4
    c.commit_chunk(alloc["chunk_key"])
    assert c.lookup(toks, "m")[0]["chunk_key"] == alloc["chunk_key"]
    assert c.lookup_chunks([alloc["chunk_key"]], "m")[0]["token_count"] == 64
    with pytest.raises(RuntimeError, match="IPC error"):
        c.commit_chunk("missing")
    c.evict_chunk(alloc["chunk_key"])
    c.close()


def test_async_client(live_plane):
    import asyncio

    async def go():
        c = IPCClientAsync(live_plane.socket_path)
        s = IPCClientSync(live_plane.socket_path)
        loop = asyncio.get_running_loop()
        await loop.run_in_executor(None, s.alloc_chunk, "ak", 16, "m")
        await c.commit_chunk("ak")
        r = await c.register_doc("doc", "title", ["ak"], 16, tokens=list(range(16)))
        assert r["chunk_count_cached"] == 1
        assert (await c.list_docs())[0]["doc_id"] == "doc"
        assert (await c.get_doc("doc"))["title"] == "title"
        assert (await c.evict_doc("doc"))["chunks_evicted"] == 1
        await c.close()
        s.close()

    asyncio.run(go())


def test_packed_token_ids_are_negotiated_and_equivalent(live_plane):
    """`hello` advertises `tokens_bin`; lookups with packed int32 ids answer like lists do, and a
    client that never negotiates keeps the reference's wire form."""
    from daser_b200.connector.ipc_client import IPCClientSync

    p = live_plane.socket_path
    plain, packed = IPCClientSync(p), IPCClientSync(p)
    try:
        assert packed.negotiate() is True and packed.binary_tokens and not plain.binary_tokens
        toks = list(range(1000, 1000 + 70))
        key = hash_tokens(toks[:64])
        chunks, alloc = packed.match_and_alloc(toks, key, "m")
        assert chunks == [] and alloc["token_count"] == 64
        packed.commit_chunk(key)
        for c in (plain, packed):
            got = c.lookup(toks + [1, 2, 3], "m")
            assert len(got) == 1 and got[0]["chunk_key"] == key
            assert c.lookup(toks[:10], "m") == []
        assert rpc(p, {"op": "lookup", "tokens_bin": b"\x01\x02\x03", "model_id": "m"}).get("error")
    finally:
        plain.close()
        packed.close()


def test_ring_occupancy_gauges_follow_the_ring(live_plane):
    from daser_b200 import metrics

    p = live_plane.socket_path
    rpc(p, {"op": "alloc_chunk", "chunk_key": "g1", "token_count": 40, "model_id": "m"})
    snap = metrics.snapshot()
    assert snap["ring.used_slots"] == 3 and snap["ring.chunks"] == 1 and snap["ring.total_slots"] >= 3
    rpc(p, {"op": "commit_chunk", "chunk_key": "g1"})
    rpc(p, {"op": "evict_chunk", "chunk_key": "g1"})
    assert metrics.snapshot()["ring.chunks"] == 0
    assert "daser_ring_used_slots" in metrics.prometheus_text()
