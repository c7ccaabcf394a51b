"""RPC clients for the control plane.

Capability parity: ``daser/connector/ipc_client.py:53-317``.

* :class:`IPCClientSync` — blocking, one persistent socket, 30 s timeout, a
  lock around each exchange, one reconnect-and-retry on a transport failure,
  ``RuntimeError`` on transport failure or an ``{"error": ...}`` reply.
  Methods: ``call, close, lookup, match_and_alloc, alloc_chunk, commit_chunk,
  evict_chunk`` plus the additions ``lookup_chunks, abort_chunk, hello,
  stats``.
* :class:`IPCClientAsync` — asyncio.  The reference opens a new connection per
  call (``ipc_client.py:228-240``); this one keeps a connection per event loop
  and falls back to reconnecting once.  Methods: ``call, commit_chunk,
  register_doc, list_docs, get_doc, evict_doc`` plus ``lookup_chunks``.
"""

from __future__ import annotations

import asyncio
import sys
from array import array
import socket
import threading
from typing import Any, Optional

from daser_b200.proto import frames

_TIMEOUT_S = 30.0


class IPCClientSync:
    def __init__(self, socket_path: str, timeout: float = _TIMEOUT_S) -> None:
        self._path = socket_path
        self._timeout = timeout
        self._sock: Optional[socket.socket] = None
        self._lock = threading.Lock()
        # token ids travel as a msgpack list (the reference's wire form) until `negotiate` finds
        # a server that also takes them as packed int32 (one bin field instead of n integers)
        self.binary_tokens = False
        self._fast: Optional["IPCClientSync"] = None  # client of the server's native lookup socket
        self.negotiated = False  # a server has answered `negotiate` (with its features, or with "unknown op")

    def negotiate(self) -> bool:
        """Ask the server what it supports; enables packed token ids when it does.  A server
        without the ``hello`` operation (the reference's) leaves everything as it is."""
        try:
            reply = self.call({"op": frames.OP_HELLO, "geometry": {}})
        except RuntimeError as exc:
            # a server that answered "unknown op" has been asked; one that could not be reached has not
            self.negotiated = "IPC error from server" in str(exc)
            return False
        self.negotiated = True
        self.binary_tokens = "tokens_bin" in (reply.get("features") or [])
        # lookups by key may go to the server's native thread, on a socket of its own
        fast = reply.get("fast_lookup")
        if isinstance(fast, str) and fast and fast != self._path:
            self._fast = IPCClientSync(fast, timeout=self._timeout)
        return self.binary_tokens

    def _tok(self, tokens) -> dict[str, Any]:
        if self.binary_tokens:
            buf = tokens if isinstance(tokens, array) and tokens.typecode == "i" else array("i", tokens)
            if sys.byteorder != "little":  # pragma: no cover
                buf = array("i", buf)
                buf.byteswap()
            return {"tokens_bin": buf.tobytes()}
        return {"tokens": list(tokens)}

    def _connect(self) -> socket.socket:
        if self._sock is None:
            s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            s.settimeout(self._timeout)
            try:
                s.connect(self._path)
            except OSError:
                s.close()
                raise
            self._sock = s
        return self._sock

    def _reset(self) -> None:
        if self._sock is not None:
            try:
                self._sock.close()
            except OSError:
                pass
            self._sock = None

    def call(self, payload: dict[str, Any]) -> dict[str, Any]:
        data = frames.pack(payload)
        last: Optional[BaseException] = None
        with self._lock:
            for _attempt in range(2):
                try:
                    sock = self._connect()
                    sock.sendall(data)
                    reply = frames.recv_frame(sock)
                    break
                except (ConnectionError, OSError) as exc:
                    last = exc
                    self._reset()
            else:
                raise RuntimeError(
                    f"IPC call {payload.get('op')!r} failed: {last!r}"
                ) from last
        if "error" in reply:
            raise RuntimeError(f"IPC error from server: {reply['error']}")
        return reply

    def close(self) -> None:
        with self._lock:
            self._reset()
        if self._fast is not None:
            self._fast.close()
            self._fast = None

    # reference operations
    def lookup(self, tokens: list[int], model_id: str) -> list[dict[str, Any]]:
        return self.call({"op": frames.OP_LOOKUP, **self._tok(tokens), "model_id": model_id})[
            "chunks"
        ]

    def match_and_alloc(
        self, tokens: list[int], chunk_key: str, model_id: str
    ) -> tuple[list[dict[str, Any]], Optional[dict[str, Any]]]:
        reply = self.call(
            {
                "op": frames.OP_MATCH_AND_ALLOC,
                **self._tok(tokens),
                "chunk_key": chunk_key,
                "model_id": model_id,
            }
        )
        return reply.get("chunks", []), reply.get("alloc")

    def alloc_chunk(self, chunk_key: str, token_count: int, model_id: str,
                    pos_offset: Optional[int] = None) -> dict[str, Any]:
        payload: dict[str, Any] = {
            "op": frames.OP_ALLOC_CHUNK,
            "chunk_key": chunk_key,
            "token_count": token_count,
            "model_id": model_id,
        }
        if pos_offset is not None:
            payload["pos_offset"] = pos_offset
        return self.call(payload)

    def commit_chunk(self, chunk_key: str, **extra: Any) -> None:
        self.call({"op": frames.OP_COMMIT_CHUNK, "chunk_key": chunk_key, **extra})

    def evict_chunk(self, chunk_key: str) -> None:
        self.call({"op": frames.OP_EVICT_CHUNK, "chunk_key": chunk_key})

    # additions
    def lookup_chunks(
        self, keys: list[str], model_id: str
    ) -> list[Optional[dict[str, Any]]]:
        msg = {"op": frames.OP_LOOKUP_CHUNKS, "keys": keys, "model_id": model_id}
        if self._fast is not None:
            try:
                return self._fast.call(msg)["chunks"]
            except (RuntimeError, OSError, KeyError):  # the thread went away: the main socket still answers
                self._fast.close()
                self._fast = None
        return self.call(msg)["chunks"]

    def scan_chunks(self, tokens: list[int], model_id: str) -> list[dict[str, Any]]:
        return self.call(
            {"op": frames.OP_LOOKUP_CHUNKS, **self._tok(tokens), "model_id": model_id}
        )["hits"]

    def abort_chunk(self, chunk_key: str) -> bool:
        return bool(
            self.call({"op": frames.OP_ABORT_CHUNK, "chunk_key": chunk_key}).get("released")
        )

    def hello(self, geometry: dict[str, Any]) -> dict[str, Any]:
        return self.call({"op": frames.OP_HELLO, "geometry": geometry})

    def stats(self) -> dict[str, Any]:
        return self.call({"op": frames.OP_STATS})


class IPCClientAsync:
    def __init__(self, socket_path: str, timeout: float = _TIMEOUT_S) -> None:
        self._path = socket_path
        self._timeout = timeout
        self._conn: Optional[tuple[asyncio.AbstractEventLoop, Any, Any]] = None
        self._lock: Optional[asyncio.Lock] = None

    async def _streams(self):
        loop = asyncio.get_running_loop()
        if self._conn is not None and self._conn[0] is loop:
            return self._conn[1], self._conn[2]
        await self._drop()
        reader, writer = await asyncio.wait_for(
            asyncio.open_unix_connection(self._path), self._timeout
        )
        self._conn = (loop, reader, writer)
        return reader, writer

    async def _drop(self) -> None:
        if self._conn is not None:
            _, _, writer = self._conn
            self._conn = None
            try:
                writer.close()
            except Exception:
                pass

    async def call(self, payload: dict[str, Any]) -> dict[str, Any]:
        loop = asyncio.get_running_loop()
        if self._lock is None or getattr(self._lock, "_daser_loop", None) is not loop:
            self._lock = asyncio.Lock()
            self._lock._daser_loop = loop  # type: ignore[attr-defined]
        last: Optional[BaseException] = None
        async with self._lock:
            for _attempt in range(2):
                try:
                    reader, writer = await self._streams()
                    await frames.write_frame(writer, payload)
                    reply = await asyncio.wait_for(
                        frames.read_frame(reader), self._timeout
                    )
                    break
                except (
                    ConnectionError,
                    OSError,
                    asyncio.IncompleteReadError,
                    asyncio.TimeoutError,
                ) as exc:
                    last = exc
                    await self._drop()
            else:
                raise RuntimeError(
                    f"IPC call {payload.get('op')!r} failed: {last!r}"
                ) from last
        if "error" in reply:
            raise RuntimeError(f"IPC error from server: {reply['error']}")
        return reply

    async def close(self) -> None:
        await self._drop()

    async def commit_chunk(self, chunk_key: str, **extra: Any) -> None:
        await self.call({"op": frames.OP_COMMIT_CHUNK, "chunk_key": chunk_key, **extra})

    async def register_doc(
        self,
        doc_id: str,
        title: str,
        chunk_keys: list[str],
        token_count: int,
        tokens: Optional[list[int]] = None,
    ) -> dict[str, Any]:
        payload: dict[str, Any] = {
            "op": frames.OP_REGISTER_DOC,
            "doc_id": doc_id,
            "title": title,
            "chunk_keys": chunk_keys,
            "token_count": token_count,
        }
        if tokens is not None:
            payload["tokens"] = tokens
        return await self.call(payload)

    async def list_docs(self) -> list[dict[str, Any]]:
        return (await self.call({"op": frames.OP_LIST_DOCS}))["docs"]

    async def get_doc(self, doc_id: str) -> dict[str, Any]:
        return (await self.call({"op": frames.OP_GET_DOC, "doc_id": doc_id}))["doc"]

    async def evict_doc(self, doc_id: str) -> dict[str, Any]:
        return await self.call({"op": frames.OP_EVICT_DOC, "doc_id": doc_id})

    async def lookup_chunks(
        self, keys: list[str], model_id: str
    ) -> list[Optional[dict[str, Any]]]:
        reply = await self.call(
            {"op": frames.OP_LOOKUP_CHUNKS, "keys": keys, "model_id": model_id}
        )
        return reply["chunks"]

    async def stats(self) -> dict[str, Any]:
        return await self.call({"op": frames.OP_STATS})
