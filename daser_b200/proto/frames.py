"""Wire framing shared by the RPC clients and the server.

Frame = 4-byte big-endian payload length + msgpack map (``use_bin_type=True``
when packing, ``raw=False`` when unpacking), exactly as in
``daser/connector/ipc_client.py:17-50`` and ``daser/server/ipc_server.py:21-49``.
The reference repeats these helpers on both sides; this module is the single
definition.  A frame longer than :data:`MAX_FRAME` is rejected before any
allocation, so a corrupted length prefix cannot make the server allocate GBs.
"""

from __future__ import annotations

import asyncio
import socket
import struct
from typing import Any

import msgpack

HEADER = struct.Struct(">I")
MAX_FRAME = 512 * 1024 * 1024

# The nine operations of the reference protocol.
OP_LOOKUP = "lookup"
OP_ALLOC_CHUNK = "alloc_chunk"
OP_MATCH_AND_ALLOC = "match_and_alloc"
OP_COMMIT_CHUNK = "commit_chunk"
OP_EVICT_CHUNK = "evict_chunk"
OP_REGISTER_DOC = "register_doc"
OP_LIST_DOCS = "list_docs"
OP_GET_DOC = "get_doc"
OP_EVICT_DOC = "evict_doc"
# Additions (absent from the reference).
OP_LOOKUP_CHUNKS = "lookup_chunks"
OP_ABORT_CHUNK = "abort_chunk"
OP_HELLO = "hello"
OP_STATS = "stats"

REFERENCE_OPS = (
    OP_LOOKUP,
    OP_ALLOC_CHUNK,
    OP_MATCH_AND_ALLOC,
    OP_COMMIT_CHUNK,
    OP_EVICT_CHUNK,
    OP_REGISTER_DOC,
    OP_LIST_DOCS,
    OP_GET_DOC,
    OP_EVICT_DOC,
)


class FrameError(ConnectionError):
    """Malformed, truncated or oversized frame."""


def pack(payload: dict[str, Any]) -> bytes:
    body = msgpack.packb(payload, use_bin_type=True)
    return HEADER.pack(len(body)) + body


def unpack_body(body: bytes) -> dict[str, Any]:
    try:
        msg = msgpack.unpackb(body, raw=False)
    except Exception as exc:  # msgpack raises several unrelated types
        raise FrameError(f"undecodable msgpack body: {exc}") from exc
    if not isinstance(msg, dict):
        raise FrameError("frame body is not a map")
    return msg


def _check_len(n: int) -> int:
    if n > MAX_FRAME:
        raise FrameError(f"frame of {n} bytes exceeds limit {MAX_FRAME}")
    return n


def recv_exact(sock: socket.socket, n: int) -> bytes:
    """Read exactly ``n`` bytes from a blocking socket."""
    chunks = bytearray()
    while len(chunks) < n:
        part = sock.recv(n - len(chunks))
        if not part:
            raise FrameError("socket closed mid-frame")
        chunks += part
    return bytes(chunks)


def recv_frame(sock: socket.socket) -> dict[str, Any]:
    (n,) = HEADER.unpack(recv_exact(sock, HEADER.size))
    return unpack_body(recv_exact(sock, _check_len(n)))


async def read_frame(reader: asyncio.StreamReader) -> dict[str, Any]:
    """Read one frame; ``asyncio.IncompleteReadError`` signals a clean EOF."""
    (n,) = HEADER.unpack(await reader.readexactly(HEADER.size))
    return unpack_body(await reader.readexactly(_check_len(n)))


async def write_frame(writer: asyncio.StreamWriter, payload: dict[str, Any]) -> None:
    writer.write(pack(payload))
    await writer.drain()
