"""Control-plane RPC server on a Unix socket.

Capability parity: ``daser/server/ipc_server.py:52-479`` — the nine operations
``lookup``, ``alloc_chunk``, ``match_and_alloc``, ``commit_chunk``,
``evict_chunk``, ``register_doc``, ``list_docs``, ``get_doc``, ``evict_doc``
with the same request/reply maps, ``file_offset = start_slot * slot_size``,
two-phase visibility (allocated chunks are invisible to lookups until
committed), ``{"error": str}`` replies and ``unknown op: X``.

Differences:

* A handler error that is part of the protocol (unknown key, duplicate doc)
  is answered on the same connection; only a broken frame closes it.  The
  reference closes the connection after *any* handler exception, which turns a
  duplicate allocation into a transport error on the client
  (``ipc_server.py:156-164``).
* Ring eviction invalidates the retrieval index through the allocator's
  eviction listener.
* New operations: ``lookup_chunks`` (batched lookup by key, plus an optional
  scan of a prompt for chunks at block-aligned offsets), ``abort_chunk``,
  ``hello`` (geometry handshake) and ``stats``.
* ``commit_chunk`` accepts an optional ``first_block`` digest (anchor for the
  offset scan) and ``checksum``.
"""

from __future__ import annotations

import asyncio
import sys
from array import array
import os
from typing import Any, Awaitable, Callable, Optional

from daser_b200 import metrics
from daser_b200.config import geometry_mismatch
from daser_b200.logging import init_logger
from daser_b200.position.base import PositionEncoder
from daser_b200.proto import frames
from daser_b200.retrieval.base import RetrievalIndex
from daser_b200.server.chunk_manager import ChunkManager
from daser_b200.server.doc_registry import DocEntry, DocRegistry
from daser_b200.server.metadata_store import ChunkMeta

logger = init_logger(__name__)

Handler = Callable[[dict[str, Any]], Awaitable[dict[str, Any]]]


class ProtocolError(Exception):
    """An error the client should see as ``{"error": ...}`` without losing the socket."""


class IPCServer:
    def __init__(
        self,
        socket_path: str,
        chunk_manager: ChunkManager,
        retrieval_index: RetrievalIndex,
        position_encoder: PositionEncoder,
        slot_size: int,
        block_tokens: int = 16,
        doc_registry: Optional[DocRegistry] = None,
        geometry: Optional[dict[str, Any]] = None,
        fast_lookup: Optional[bool] = None,
    ) -> None:
        # lookups by key are also served by a native thread on `<socket>.fast` (no interpreter on
        # that path); off with fast_lookup=False or DASER_FAST_LOOKUP=0
        if fast_lookup is None:
            fast_lookup = os.environ.get("DASER_FAST_LOOKUP", "1") != "0"
        self._fast_enabled = bool(fast_lookup)
        self._fast: Any = None
        self._socket_path = socket_path
        self._cm = chunk_manager
        self._ri = retrieval_index
        self._pe = position_encoder
        self._slot_size = slot_size
        self._block_tokens = block_tokens
        self._docs = doc_registry
        self._geometry = dict(geometry or {})
        self._geometry.setdefault("slot_size", slot_size)
        self._geometry.setdefault("block_tokens", block_tokens)
        self._server: Optional[asyncio.AbstractServer] = None
        self._writers: set[asyncio.StreamWriter] = set()
        self._parts: dict[str, set[int]] = {}
        self._dirty = False
        self._cm.add_eviction_listener(self._on_evicted)
        self._handlers: dict[str, Handler] = {
            frames.OP_LOOKUP: self._handle_lookup,
            frames.OP_ALLOC_CHUNK: self._handle_alloc_chunk,
            frames.OP_MATCH_AND_ALLOC: self._handle_match_and_alloc,
            frames.OP_COMMIT_CHUNK: self._handle_commit_chunk,
            frames.OP_EVICT_CHUNK: self._handle_evict_chunk,
            frames.OP_REGISTER_DOC: self._handle_register_doc,
            frames.OP_LIST_DOCS: self._handle_list_docs,
            frames.OP_GET_DOC: self._handle_get_doc,
            frames.OP_EVICT_DOC: self._handle_evict_doc,
            frames.OP_LOOKUP_CHUNKS: self._handle_lookup_chunks,
            frames.OP_ABORT_CHUNK: self._handle_abort_chunk,
            frames.OP_HELLO: self._handle_hello,
            frames.OP_STATS: self._handle_stats,
        }

    # -- lifecycle ------------------------------------------------------------

    @property
    def socket_path(self) -> str:
        return self._socket_path

    @property
    def dirty(self) -> bool:
        """True when state changed since :meth:`clear_dirty` (drives snapshots)."""
        return self._dirty

    def clear_dirty(self) -> None:
        self._dirty = False

    async def start(self) -> None:
        if os.path.exists(self._socket_path):
            os.unlink(self._socket_path)
        self._server = await asyncio.start_unix_server(
            self._handle_connection, path=self._socket_path
        )
        logger.info("[IPC] listening on %s", self._socket_path)
        self._start_fast()

    def _start_fast(self) -> None:
        from daser_b200.server.native_index import FastLookupServer

        if not self._fast_enabled or not FastLookupServer.supported():
            return
        try:
            self._fast = FastLookupServer(self._socket_path + ".fast", self._slot_size)
        except (OSError, RuntimeError) as exc:
            logger.warning("[IPC] no native lookup thread (%s): lookups stay on the main socket", exc)
            return
        for meta in self._cm.store.iter_chunks():  # what a snapshot brought back
            if self._cm.store.is_committed(meta.chunk_key):
                self._fast_put(meta)
        logger.info("[IPC] native lookup thread on %s", self._fast.socket_path)

    def _fast_put(self, meta: ChunkMeta) -> None:
        if self._fast is not None:
            self._fast.put(meta.chunk_key, meta.model_id, meta.start_slot, meta.num_slots, meta.token_count,
                           int(self._pe.get_offset(meta)))

    async def stop(self) -> None:
        if self._fast is not None:
            self._fast.stop()
            self._fast = None
        if self._server is not None:
            self._server.close()
            # wait_closed() also waits for live connections: hang up on them.
            for writer in list(self._writers):
                writer.close()
            await self._server.wait_closed()
            self._server = None
        if os.path.exists(self._socket_path):
            os.unlink(self._socket_path)
        logger.info("[IPC] server stopped")

    # -- connection loop --------------------------------------------------------

    async def _handle_connection(
        self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter
    ) -> None:
        self._writers.add(writer)
        try:
            while True:
                try:
                    msg = await frames.read_frame(reader)
                except asyncio.IncompleteReadError:
                    break  # peer closed
                reply = await self.dispatch(msg)
                await frames.write_frame(writer, reply)
        except (frames.FrameError, ConnectionError, OSError) as exc:
            logger.warning("[IPC] dropping connection: %s", exc)
            try:
                await frames.write_frame(writer, {"error": str(exc)})
            except Exception:
                pass
        finally:
            self._writers.discard(writer)
            writer.close()
            try:
                await writer.wait_closed()
            except Exception:
                pass

    async def dispatch(self, msg: dict[str, Any]) -> dict[str, Any]:
        """Run one request map through its handler (also usable in-process)."""
        op = msg.get("op")
        handler = self._handlers.get(op)  # type: ignore[arg-type]
        if handler is None:
            return {"error": f"unknown op: {op}"}
        metrics.inc(f"ipc.{op}")
        try:
            reply = await handler(msg)
            if self._dirty:  # occupancy gauges for /metrics and the stats of embedding processes
                metrics.set_gauge("ring.used_slots", self._cm.used_slots)
                metrics.set_gauge("ring.total_slots", self._cm.total_slots)
                metrics.set_gauge("ring.chunks", len(self._cm.store))
                if self._fast is not None:
                    for name, value in self._fast.stats().items():
                        metrics.set_gauge(f"fast_lookup.{name}", value)
            return reply
        except ProtocolError as exc:
            return {"error": str(exc)}
        except (KeyError, ValueError, TypeError) as exc:
            logger.warning("[IPC] op=%s failed: %r", op, exc)
            return {"error": f"{type(exc).__name__}: {exc}"}

    # -- helpers ------------------------------------------------------------------

    def _chunk_dict(self, meta: ChunkMeta) -> dict[str, Any]:
        return {
            "chunk_key": meta.chunk_key,
            "start_slot": meta.start_slot,
            "num_slots": meta.num_slots,
            "token_count": meta.token_count,
            "pos_offset": self._pe.get_offset(meta),
            "model_id": meta.model_id,
            "file_offset": meta.start_slot * self._slot_size,
        }

    def _slots_for(self, token_count: int) -> int:
        return -(-token_count // self._block_tokens)

    def _on_evicted(self, meta: ChunkMeta) -> None:
        if self._fast is not None:
            self._fast.delete(meta.chunk_key)
        self._ri.discard(meta.chunk_key)
        self._parts.pop(meta.chunk_key, None)
        self._dirty = True

    def _reserve(self, chunk_key: str, token_count: int, model_id: str,
                 pos_offset: Optional[int] = None) -> ChunkMeta:
        if token_count <= 0:
            raise ProtocolError("token_count must be positive")
        existing = self._cm.store.get(chunk_key)
        if existing is not None and self._cm.store.is_committed(chunk_key):
            raise ProtocolError(f"chunk_key already exists: {chunk_key}")
        if existing is not None:
            pos_offset = existing.pos_offset
        elif pos_offset is None:
            pos_offset = self._pe.assign_offset(chunk_key, token_count)
        try:
            self._cm.alloc(
                chunk_key,
                self._slots_for(token_count),
                token_count,
                model_id,
                pos_offset,
                committed=False,
            )
        except ValueError as exc:
            raise ProtocolError(str(exc)) from exc
        self._dirty = True
        meta = self._cm.store.get(chunk_key)
        assert meta is not None
        return meta

    # -- reference operations -------------------------------------------------------

    @staticmethod
    def _tokens_of(msg: dict[str, Any]):
        """The request's token ids: ``tokens`` (a list, the reference's form) or ``tokens_bin``
        (the same ids as packed little-endian int32: no per-token msgpack object on either side)."""
        raw = msg.get("tokens_bin")
        if raw is not None:
            if len(raw) % 4:
                raise ProtocolError("tokens_bin is not a whole number of int32")
            arr = array("i")
            arr.frombytes(bytes(raw))
            if sys.byteorder != "little":  # pragma: no cover
                arr.byteswap()
            return arr
        return list(msg["tokens"])

    async def _handle_lookup(self, msg: dict[str, Any]) -> dict[str, Any]:
        found = await self._ri.lookup(self._tokens_of(msg), msg.get("model_id", "default"))
        metrics.inc("lookup.hit" if found else "lookup.miss")
        return {"chunks": [self._chunk_dict(m) for m in found]}

    async def _handle_alloc_chunk(self, msg: dict[str, Any]) -> dict[str, Any]:
        # optional "pos_offset": the position the chunk's first token had when its KV was
        # computed (defaults to the position encoder's assignment)
        pos = msg.get("pos_offset")
        meta = self._reserve(
            msg["chunk_key"], int(msg["token_count"]), msg.get("model_id", "default"),
            int(pos) if pos is not None else None,
        )
        return {
            "start_slot": meta.start_slot,
            "num_slots": meta.num_slots,
            "file_offset": meta.start_slot * self._slot_size,
            "pos_offset": meta.pos_offset,
        }

    async def _handle_match_and_alloc(self, msg: dict[str, Any]) -> dict[str, Any]:
        tokens = self._tokens_of(msg)
        model_id = msg.get("model_id", "default")
        chunk_key = msg.get("chunk_key", "")
        found = await self._ri.lookup(tokens, model_id)
        if found:
            metrics.inc("lookup.hit")
            return {"chunks": [self._chunk_dict(m) for m in found], "alloc": None}
        metrics.inc("lookup.miss")
        aligned = (len(tokens) // self._block_tokens) * self._block_tokens
        if not chunk_key or aligned == 0:
            return {"chunks": [], "alloc": None}
        meta = self._reserve(chunk_key, aligned, model_id)
        return {
            "chunks": [],
            "alloc": {
                "chunk_key": chunk_key,
                "start_slot": meta.start_slot,
                "num_slots": meta.num_slots,
                "file_offset": meta.start_slot * self._slot_size,
                "pos_offset": meta.pos_offset,
                "token_count": aligned,
            },
        }

    async def _handle_commit_chunk(self, msg: dict[str, Any]) -> dict[str, Any]:
        chunk_key = msg["chunk_key"]
        meta = self._cm.store.get(chunk_key)
        if meta is None:
            raise ProtocolError(f"commit_chunk: unknown chunk_key {chunk_key}")
        parts = int(msg.get("parts", 1) or 1)
        if parts > 1:
            # several writers hold a piece each (tensor-parallel workers with their own files):
            # the chunk becomes visible when the last piece is in
            seen = self._parts.setdefault(chunk_key, set())
            seen.add(int(msg.get("part", 0)))
            if len(seen) < parts:
                return {"ok": True, "pending_parts": parts - len(seen)}
            self._parts.pop(chunk_key, None)
        anchor = msg.get("first_block")
        self._cm.store.mark_committed(chunk_key, msg.get("checksum"), anchor)
        await self._ri.insert(meta)
        self._fast_put(meta)  # visible on the native lookup socket before this commit is acknowledged
        if anchor and hasattr(self._ri, "register_anchor"):
            self._ri.register_anchor(chunk_key, anchor)  # type: ignore[attr-defined]
        self._dirty = True
        return {"ok": True}

    async def _handle_evict_chunk(self, msg: dict[str, Any]) -> dict[str, Any]:
        chunk_key = msg["chunk_key"]
        await self._ri.remove(chunk_key)
        self._cm.evict_chunk(chunk_key)
        self._dirty = True
        return {"ok": True}

    def _require_docs(self) -> DocRegistry:
        if self._docs is None:
            raise ProtocolError("doc registry not enabled")
        return self._docs

    async def _handle_register_doc(self, msg: dict[str, Any]) -> dict[str, Any]:
        docs = self._require_docs()
        doc_id = msg["doc_id"]
        if docs.get(doc_id) is not None:
            raise ProtocolError(f"doc_id already exists: {doc_id}")
        chunk_keys = list(msg.get("chunk_keys", []))
        mask = []
        for key in chunk_keys:
            meta = self._cm.store.get(key)
            live = meta is not None and self._cm.store.is_committed(key)
            if live and doc_id not in meta.doc_ids:  # type: ignore[union-attr]
                meta.doc_ids.append(doc_id)  # type: ignore[union-attr]
            mask.append(bool(live))
        tokens = msg.get("tokens")
        status = "ready" if any(mask) else "evicted"
        docs.insert(
            DocEntry(
                doc_id=doc_id,
                title=msg.get("title", ""),
                token_count=int(msg.get("token_count", 0)),
                chunk_keys=chunk_keys,
                cached_mask=mask,
                status=status,
                tokens=list(tokens) if tokens is not None else None,
            )
        )
        self._dirty = True
        return {"ok": True, "chunk_count_cached": sum(mask)}

    async def _handle_list_docs(self, msg: dict[str, Any]) -> dict[str, Any]:
        docs = self._require_docs()
        return {
            "docs": [
                {
                    "doc_id": e.doc_id,
                    "title": e.title,
                    "token_count": e.token_count,
                    "chunk_count_total": len(e.chunk_keys),
                    "chunk_count_cached": e.cached_count,
                    "status": e.status,
                    "created_at": e.created_at,
                }
                for e in docs.all_entries()
            ]
        }

    async def _handle_get_doc(self, msg: dict[str, Any]) -> dict[str, Any]:
        docs = self._require_docs()
        entry = docs.get(msg["doc_id"])
        if entry is None:
            raise ProtocolError(f"unknown doc_id: {msg['doc_id']}")
        return {
            "doc": {
                "doc_id": entry.doc_id,
                "title": entry.title,
                "created_at": entry.created_at,
                "token_count": entry.token_count,
                "chunk_keys": list(entry.chunk_keys),
                "cached_mask": list(entry.cached_mask),
                "status": entry.status,
                "tokens": entry.tokens,
                "error": entry.error,
            }
        }

    async def _handle_evict_doc(self, msg: dict[str, Any]) -> dict[str, Any]:
        docs = self._require_docs()
        entry = docs.remove(msg["doc_id"])
        if entry is None:
            raise ProtocolError(f"unknown doc_id: {msg['doc_id']}")
        evicted = 0
        for key in dict.fromkeys(entry.chunk_keys):
            meta = self._cm.store.get(key)
            if meta is None:
                continue
            if entry.doc_id in meta.doc_ids:
                meta.doc_ids.remove(entry.doc_id)
            if not meta.doc_ids:
                await self._ri.remove(key)
                self._cm.evict_chunk(key)
                evicted += 1
        self._dirty = True
        return {"ok": True, "chunks_evicted": evicted}

    # -- additions ------------------------------------------------------------------------

    async def _handle_lookup_chunks(self, msg: dict[str, Any]) -> dict[str, Any]:
        """``keys`` -> one entry (or None) per key; ``tokens`` -> scan hits with offsets."""
        model_id = msg.get("model_id", "default")
        out: dict[str, Any] = {}
        if "keys" in msg:
            chunks = []
            for key in msg["keys"]:
                meta = self._cm.store.get(key)
                ok = (
                    meta is not None
                    and meta.model_id == model_id
                    and self._cm.store.is_committed(key)
                )
                metrics.inc("lookup_chunks.hit" if ok else "lookup_chunks.miss")
                chunks.append(self._chunk_dict(meta) if ok else None)  # type: ignore[arg-type]
            out["chunks"] = chunks
        if "tokens" in msg or "tokens_bin" in msg:
            if not hasattr(self._ri, "scan"):
                raise ProtocolError("retrieval index does not support offset scans")
            hits = self._ri.scan(self._tokens_of(msg), model_id,  # type: ignore[attr-defined]
                                 any_offset=bool(msg.get("any_offset", False)))
            out["hits"] = [
                {**self._chunk_dict(h.meta), "offset": h.offset} for h in hits
            ]
        return out

    async def _handle_abort_chunk(self, msg: dict[str, Any]) -> dict[str, Any]:
        released = self._cm.abort(msg["chunk_key"])
        self._dirty = self._dirty or released
        return {"ok": True, "released": released}

    async def _handle_hello(self, msg: dict[str, Any]) -> dict[str, Any]:
        bad = geometry_mismatch(self._geometry, dict(msg.get("geometry") or {}))
        if bad:
            raise ProtocolError("geometry mismatch: " + "; ".join(bad))
        reply = {"ok": True, "geometry": self._geometry, "ops": sorted(self._handlers),
                 "features": ["tokens_bin"]}
        if self._fast is not None:
            reply["fast_lookup"] = self._fast.socket_path
        return reply

    async def _handle_stats(self, msg: dict[str, Any]) -> dict[str, Any]:
        return {
            "ring": {
                "total_slots": self._cm.total_slots,
                "used_slots": self._cm.used_slots,
                "head": self._cm.head,
                "tail": self._cm.tail,
                "chunks": len(self._cm.store),
            },
            "docs": len(self._docs) if self._docs is not None else 0,
            "counters": metrics.snapshot(),
            **({"fast_lookup": self._fast.stats()} if self._fast is not None else {}),
        }
