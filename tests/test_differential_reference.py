"""Differential tests against the reference's pure-Python control plane, when it is installed.

``baseline/_ref`` holds the unmodified reference (installed offline with ``--no-deps``); its
server, allocator and index import only msgpack and xxhash.  Same operations in, same answers
out; and each side's client talks to the other side's server over the real socket.
"""

import asyncio
import os
import random
import sys
import threading

import pytest

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
if not os.path.isdir(os.path.join(REF, "daser")):
    pytest.skip("reference not installed under baseline/_ref", allow_module_level=True)
sys.path.insert(0, REF)

from daser.position.fixed_offset import FixedOffsetEncoder as RefPE  # noqa: E402
from daser.retrieval.prefix import PrefixHashIndex as RefIndex  # noqa: E402
from daser.server.chunk_manager import ChunkManager as RefRing  # noqa: E402
from daser.server.doc_registry import DocRegistry as RefDocs  # noqa: E402
from daser.server.ipc_server import IPCServer as RefServer  # noqa: E402
from daser.server.metadata_store import MetadataStore as RefStore  # noqa: E402

from conftest import LiveControlPlane  # noqa: E402
from daser_b200.connector.ipc_client import IPCClientSync  # noqa: E402
from daser_b200.hashing import hash_tokens  # noqa: E402
from daser_b200.server.chunk_manager import ChunkManager  # noqa: E402
from daser_b200.server.metadata_store import MetadataStore  # noqa: E402


def test_ring_allocator_places_chunks_like_the_reference():
    rng = random.Random(0)
    for total in (8, 16, 33):
        mine = ChunkManager(total, MetadataStore(total))
        ref = RefRing(total_slots=total, metadata_store=RefStore(total_slots=total))
        for i in range(300):
            n = rng.randint(1, max(1, total // 2))
            a = mine.alloc(f"k{i}", n, n * 16, "m", 0)
            b = ref.alloc(f"k{i}", num_slots=n, token_count=n * 16, model_id="m", pos_offset=0)
            assert a == b, (total, i, n)
            live = {c.chunk_key: (c.start_slot, c.num_slots) for c in mine.store.iter_chunks()}
            # The reference can keep a chunk in its index after handing the same slots to a new
            # one (a full ring whose head wraps: free space is derived from head/tail alone, e.g.
            # total 8, chunks [0,4) and [4,7), head = tail = 7, allocating 2 slots lands on [0,2)
            # without evicting [0,4)).  So: same placements, our live set is a subset of theirs,
            # and ours never overlaps.
            assert set(live) <= {c.chunk_key for c in ref.store.iter_chunks()}
            spans = sorted(live.values())
            assert all(s0 + n0 <= s1 for (s0, n0), (s1, _) in zip(spans, spans[1:]))


def test_snapshot_written_here_loads_in_the_reference_and_back(tmp_path):
    mine = ChunkManager(16, MetadataStore(16))
    for i, n in enumerate((3, 2, 5)):
        mine.alloc(f"k{i}", n, n * 16, "m", 0)
    p = str(tmp_path / "daser.index")
    mine.save(p)
    ref = RefRing(total_slots=16, metadata_store=RefStore(total_slots=16))
    ref.load(p)
    assert (ref.head, ref.tail) == (mine.head, mine.tail) and ref.store.get("k2").start_slot == 5
    p2 = str(tmp_path / "ref.index")
    ref.save(p2)
    back = ChunkManager(16, MetadataStore(16))
    back.load(p2)
    assert back.used_slots == 10 and back.store.get("k1").num_slots == 2


def test_hashes_match():
    from daser.retrieval.prefix import _hash_tokens

    toks = [random.Random(1).randrange(150000) for _ in range(77)]
    assert hash_tokens(toks) == _hash_tokens(toks)


class _RefPlane:
    """The reference server on a thread, like its own test fixtures do."""

    def __init__(self, path):
        store = RefStore(total_slots=64)
        self.server = RefServer(path, RefRing(64, store, RefDocs()), RefIndex(16), RefPE(0), slot_size=4096,
                                block_tokens=16, doc_registry=RefDocs())
        self.loop = asyncio.new_event_loop()
        self.ready = threading.Event()
        threading.Thread(target=self._run, daemon=True).start()
        assert self.ready.wait(10)

    def _run(self):
        asyncio.set_event_loop(self.loop)
        self.loop.run_until_complete(self.server.start())
        self.ready.set()
        self.loop.run_forever()

    def stop(self):
        asyncio.run_coroutine_threadsafe(self.server.stop(), self.loop).result(10)
        self.loop.call_soon_threadsafe(self.loop.stop)


def _exercise(client, tokens):
    key = hash_tokens(tokens[:32])
    out = [client.lookup(tokens, "m")]
    chunks, alloc = client.match_and_alloc(tokens, key, "m")
    out.append((chunks, {k: alloc[k] for k in sorted(alloc)}))
    client.commit_chunk(key)
    hit = client.lookup(tokens, "m")
    out.append([{k: v for k, v in c.items()} for c in hit])
    a2 = client.alloc_chunk("other", 40, "m")
    out.append({k: a2[k] for k in sorted(a2)})
    client.evict_chunk(key)
    out.append(client.lookup(tokens, "m"))
    return out


def test_same_replies_over_the_wire_from_both_servers(tmp_path):
    tokens = list(range(500, 540))
    ref = _RefPlane(str(tmp_path / "ref.sock"))
    mine = LiveControlPlane(tmp_path).start()
    try:
        c_ref, c_mine = IPCClientSync(str(tmp_path / "ref.sock")), IPCClientSync(mine.socket_path)
        assert _exercise(c_ref, tokens) == _exercise(c_mine, tokens)
        c_ref.close(), c_mine.close()
    finally:
        ref.stop()
        mine.stop()


def test_reference_clients_talk_to_this_server(tmp_path):
    """The unmodified reference clients (sync and async) against this control plane: the wire
    protocol is the reference's, so its connector and its service can be pointed here."""
    from daser.connector.ipc_client import IPCClientAsync as RefAsync
    from daser.connector.ipc_client import IPCClientSync as RefSync

    tokens = list(range(700, 740))
    ref = _RefPlane(str(tmp_path / "ref.sock"))
    mine = LiveControlPlane(tmp_path).start()
    try:
        # same scripted session through the reference's own sync client, on both servers
        def session(client):
            key = hash_tokens(tokens[:32])
            out = [client.call({"op": "lookup", "tokens": tokens, "model_id": "m"})]
            out.append(client.call({"op": "match_and_alloc", "tokens": tokens, "chunk_key": key, "model_id": "m"}))
            out.append(client.call({"op": "commit_chunk", "chunk_key": key}))
            out.append(client.call({"op": "lookup", "tokens": tokens + [9], "model_id": "m"}))
            out.append(client.call({"op": "alloc_chunk", "chunk_key": "other", "token_count": 40, "model_id": "m"}))
            out.append(client.call({"op": "evict_chunk", "chunk_key": key}))
            out.append(client.call({"op": "lookup", "tokens": tokens, "model_id": "m"}))
            return out

        a, b = RefSync(str(tmp_path / "ref.sock")), RefSync(mine.socket_path)
        try:
            got_a, got_b = session(a), session(b)
        finally:
            a.close(), b.close()
        # this server adds fields the reference's replies do not have; what the reference sends must match
        for ra, rb in zip(got_a, got_b):
            assert set(ra) <= set(rb), (ra, rb)  # every field of the reference's reply is present here
            for k in ra:
                va, vb = ra[k], rb[k]
                if isinstance(va, list) and va and isinstance(va[0], dict):
                    assert [{f: d[f] for f in va[i]} for i, d in enumerate(vb)] == va
                elif isinstance(va, dict):
                    assert {f: vb[f] for f in va} == va
                else:
                    assert va == vb

        async def docs(path):
            c = RefAsync(path)
            key = hash_tokens(list(range(16)))
            sync = IPCClientSync(path)
            sync.alloc_chunk(key, 16, "m")
            await c.commit_chunk(key)
            r = await c.register_doc("d1", "Title", [key, "missing"], 32, list(range(32)))
            listing = await c.list_docs()
            doc = await c.get_doc("d1")
            gone = await c.evict_doc("d1")
            after = await c.list_docs()
            sync.close()
            for d in listing + [doc]:
                d.pop("created_at", None)
            return r, listing, doc, gone, after

        got_ref = asyncio.run(docs(str(tmp_path / "ref.sock")))
        got_mine = asyncio.run(docs(mine.socket_path))
        assert got_ref == got_mine
    finally:
        ref.stop()
        mine.stop()
