"""Frozen bytes of the three formats a deployment cannot change under its users: the RPC frames,
the store file's slot image (``raw`` codec) and the snapshot.

The expected bytes are spelled out by hand from the format descriptions
(``daser/connector/ipc_client.py:17-28`` and ``daser/server/ipc_server.py:21-49`` for frames,
``daser/connector/daser_connector.py:625-632`` for slots, ``daser/server/chunk_manager.py:201-210``
and ``daser/server/metadata_store.py:207-216`` for snapshots), not produced by the code under test.
"""

import socket
import struct

import msgpack
import torch

from conftest import LiveControlPlane
from daser_b200.connector.core import TorchKVBackend
from daser_b200.kv.layout import KVGeometry
from daser_b200.proto import frames


def _fixstr(s: str) -> bytes:
    assert len(s) < 32
    return bytes([0xA0 | len(s)]) + s.encode()


def test_request_frame_bytes_are_the_references():
    # {"op": "alloc_chunk", "chunk_key": "ab", "token_count": 32, "model_id": "m"}
    body = (b"\x84" + _fixstr("op") + _fixstr("alloc_chunk") + _fixstr("chunk_key") + _fixstr("ab")
            + _fixstr("token_count") + b"\x20" + _fixstr("model_id") + _fixstr("m"))
    golden = struct.pack(">I", len(body)) + body
    msg = {"op": "alloc_chunk", "chunk_key": "ab", "token_count": 32, "model_id": "m"}
    assert frames.pack(msg) == golden
    # token ids above 127 use the shortest msgpack integer form; lists keep their order
    body = b"\x82" + _fixstr("op") + _fixstr("lookup") + _fixstr("tokens") + b"\x93\x7f\xcc\x80\xcd\x7d\x00"
    assert frames.pack({"op": "lookup", "tokens": [127, 128, 32000]}) == struct.pack(">I", len(body)) + body


def test_server_replies_byte_for_byte(tmp_path):
    lp = LiveControlPlane(tmp_path, total_slots=8, slot_size=4096).start()
    try:
        s = socket.socket(socket.AF_UNIX)
        s.connect(lp.socket_path)

        def rpc(raw_body: bytes) -> bytes:
            s.sendall(struct.pack(">I", len(raw_body)) + raw_body)
            n = struct.unpack(">I", s.recv(4, socket.MSG_WAITALL))[0]
            return s.recv(n, socket.MSG_WAITALL)

        req = (b"\x84" + _fixstr("op") + _fixstr("alloc_chunk") + _fixstr("chunk_key") + _fixstr("ab")
               + _fixstr("token_count") + b"\x20" + _fixstr("model_id") + _fixstr("m"))
        # {"start_slot": 0, "num_slots": 2, "file_offset": 0, "pos_offset": 0}
        assert rpc(req) == (b"\x84" + _fixstr("start_slot") + b"\x00" + _fixstr("num_slots") + b"\x02"
                            + _fixstr("file_offset") + b"\x00" + _fixstr("pos_offset") + b"\x00")
        req = b"\x82" + _fixstr("op") + _fixstr("commit_chunk") + _fixstr("chunk_key") + _fixstr("ab")
        assert rpc(req) == b"\x81" + _fixstr("ok") + b"\xc3"
        # a second chunk lands behind the first: file_offset = start_slot * slot_size = 2 * 4096
        req = (b"\x84" + _fixstr("op") + _fixstr("alloc_chunk") + _fixstr("chunk_key") + _fixstr("cd")
               + _fixstr("token_count") + b"\x10" + _fixstr("model_id") + _fixstr("m"))
        assert rpc(req) == (b"\x84" + _fixstr("start_slot") + b"\x02" + _fixstr("num_slots") + b"\x01"
                            + _fixstr("file_offset") + b"\xcd\x20\x00" + _fixstr("pos_offset") + b"\x00")
        req = b"\x81" + _fixstr("op") + _fixstr("bogus")
        assert rpc(req) == b"\x81" + _fixstr("error") + _fixstr("unknown op: bogus")
        s.close()
    finally:
        lp.stop()


def test_raw_slot_image_layout_is_layer_kv_token_head_dim():
    """Element (layer l, K|V s, token t, head h, dim d) of a block sits at byte
    ``l * layer_size + (((s * B + t) * H + h) * D + d) * dtype_bytes`` of its slot."""
    L, H, D, B = 2, 2, 4, 16
    geo = KVGeometry(L, H, D, B, 2, "raw")
    assert geo.slot_size == H * D * 2 * L * B * 2 and geo.layer_size == geo.slot_size // L
    # pool [L, N, 2, H, B, D]; value encodes its own coordinates (exact in bf16: < 256)
    pool = torch.zeros(L, 3, 2, H, B, D, dtype=torch.bfloat16)
    for l in range(L):
        for s in range(2):
            for h in range(H):
                for t in range(B):
                    pool[l, 1, s, h, t] = torch.tensor([l * 128 + s * 64 + h * 32 + t * 2 + (d & 1) for d in range(D)],
                                                      dtype=torch.bfloat16)
    image = torch.zeros(1, geo.slot_size, dtype=torch.uint8)
    TorchKVBackend(geo, pool, [1.0] * (D // 2)).save([1], image)
    raw = image[0].numpy().tobytes()
    for (l, s, t, h, d) in [(0, 0, 0, 0, 0), (0, 0, 0, 0, 1), (0, 0, 1, 0, 0), (0, 0, 0, 1, 0), (0, 1, 0, 0, 0),
                            (1, 0, 0, 0, 0), (1, 1, 15, 1, 3)]:
        off = l * geo.layer_size + (((s * B + t) * H + h) * D + d) * 2
        want = torch.tensor([l * 128 + s * 64 + h * 32 + t * 2 + (d & 1)], dtype=torch.bfloat16).view(torch.int16).item()
        assert struct.unpack_from("<h", raw, off)[0] == want, (l, s, t, h, d)
    # and back: restoring the image into another block reproduces the block
    TorchKVBackend(geo, pool, [1.0] * (D // 2)).restore(image, [2], [0])
    assert torch.equal(pool[:, 2], pool[:, 1])


def test_a_snapshot_in_the_references_format_loads(tmp_path):
    """A hand-built ``daser.index`` with exactly the reference's fields (no ``committed`` flag, no
    checksums): one 2-slot chunk at slot 1 of 4, head 3, tail 1."""
    chunk = {"chunk_key": "k1", "start_slot": 1, "num_slots": 2, "token_count": 32, "pos_offset": 0,
             "model_id": "m", "created_at": 1.0, "doc_ids": []}
    slot_map = [{"kind": "empty", "chunk_key": None, "num_slots": 0},
                {"kind": "chunk", "chunk_key": "k1", "num_slots": 2},
                {"kind": "cont", "chunk_key": "k1", "num_slots": 0},
                {"kind": "empty", "chunk_key": None, "num_slots": 0}]
    index = msgpack.packb({"total_slots": 4, "chunk_index": {"k1": chunk}, "slot_map": slot_map}, use_bin_type=True)
    snap = msgpack.packb({"head": 3, "tail": 1, "index": index, "doc_registry": {}}, use_bin_type=True)
    (tmp_path / "daser.index").write_bytes(snap)
    lp = LiveControlPlane(tmp_path, total_slots=4, slot_size=4096).start()
    try:
        from daser_b200.connector.ipc_client import IPCClientSync

        c = IPCClientSync(lp.socket_path)
        got = c.lookup_chunks(["k1"], "m")[0]
        assert got is not None and got["start_slot"] == 1 and got["num_slots"] == 2 and got["file_offset"] == 4096
        st = c.stats()["ring"]
        assert (st["head"], st["tail"], st["used_slots"]) == (3, 1, 2)
        c.close()
    finally:
        lp.stop()


def test_slot_sizes_of_the_models_the_reference_names():
    """``heads * hd * 2 * L * B * dtype_bytes`` (``daser/config.py:68-75``): 2 359 296 bytes for
    Qwen3-8B (``tests/integration/conftest.py:30`` there), 2 MiB for the Llama-3-8B-like geometry
    of its storage benchmark (``benchmarks/bench_storage_imdb.py:47-48``)."""
    from daser_b200.models.llama import PRESETS

    q = PRESETS["qwen3-8b"]
    assert KVGeometry(q.num_layers, q.num_kv_heads, q.head_dim, q.block_tokens, 2, "raw").slot_size == 2_359_296
    m = PRESETS["llama3-8b"]
    assert KVGeometry(m.num_layers, m.num_kv_heads, m.head_dim, m.block_tokens, 2, "raw").slot_size == 2_097_152
