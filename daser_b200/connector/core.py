"""Engine-agnostic connector: the scheduler half and the worker half.

Capability parity: ``daser/connector/daser_connector.py:60-710`` — the metadata types
(``ReqLoadSpec``, ``ReqStoreSpec``, per-step metadata), the scheduler-role hooks
(``get_num_new_matched_tokens``, ``update_state_after_alloc``, ``build_connector_meta``,
``request_finished``) and the worker-role hooks (``register_kv_caches``,
``bind/clear_connector_metadata``, ``start_load_kv``, ``wait_for_layer_load``,
``save_kv_layer``, ``wait_for_save``, ``shutdown``).  The vLLM adapter
(:mod:`daser_b200.connector.daser_connector`) and the native engine both drive these
classes; nothing here imports vLLM.

What changed relative to the reference:

* Loads and saves are ONE fused kernel launch per step (``ops/csrc/kv_paged.cu``) driven by
  a device work list, instead of ``requests x slots x layers`` strided copies.
* Chunk-level reuse: a request may carry ``chunk_placements`` — (chunk_key, token offset)
  pairs — which are resolved with the batched ``lookup_chunks`` RPC and restored at their
  new positions; the kernel rotates cached keys by ``new offset - stored pos_offset``.
  The reference can only reuse exact prompt prefixes.
* Partial prefix hits honour ``num_computed_tokens`` (``skip_slots``) instead of assuming 0.
* A failed load is reported through ``take_load_errors`` so the engine recomputes; a
  reservation whose request finishes without a store is aborted.
* Staging memory is persistent (pinned host or device arena), never allocated per step; a chunk
  longer than the arena passes through it in pieces, on the way out and on the way back.
* An optional HBM tier (:mod:`daser_b200.kv.hbm_store`) serves hot chunks without IO; a pinned host
  tier of the same class sits between it and the file.
* A load can be cut by layer group (``begin_load / restore_group / end_load``): reads go out at once,
  group-major, and piece g is restored when ITS reads are in (``reads_done`` tells an engine whether
  anything is still in flight without waiting for it).
* ``write_behind`` (opt-in): ``wait_for_save`` returns with the file writes in flight; the chunk is
  committed when they are done (the reference writes and commits inside ``wait_for_save``,
  ``daser/connector/daser_connector.py:634-700``).
"""

from __future__ import annotations

import os
from collections import OrderedDict
import threading
import time
import dataclasses
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

import torch

from daser_b200 import metrics
from daser_b200.config import CODEC_FP8B16
from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.hashing import hash_tokens, prefix_digests
from daser_b200.io.engine import preallocate
from daser_b200.kv import codec
from daser_b200.kv.layout import KVGeometry, tp_head_range
from daser_b200.logging import init_logger, init_perf_logger
from daser_b200.utils import trace

logger = init_logger(__name__)
_perf = init_perf_logger("connector")


@dataclass
class ReqLoadSpec:
    """One chunk to restore into a request's blocks."""

    chunk_key: str
    start_slot: int
    num_slots: int
    block_ids: list[int]
    file_offset: int
    token_count: int
    # additions
    pos_offset: int = 0  # position the stored keys are rotated to
    dst_token_offset: int = 0  # position of the chunk's first token in this request
    skip_slots: int = 0  # leading slots the engine already has (num_computed_tokens)
    req_id: str = ""

    @property
    def delta(self) -> int:
        return self.dst_token_offset - self.pos_offset


@dataclass
class ReqStoreSpec:
    """One chunk to write from a request's blocks."""

    chunk_key: str
    start_slot: int
    num_slots: int
    block_ids: list[int]
    file_offset: int
    token_count: int
    pos_offset: int = 0
    first_block_digest: str = ""
    req_id: str = ""


@dataclass
class ConnectorMeta:
    """What the scheduler half hands to the worker half for one engine step."""

    reqs_to_load: list[ReqLoadSpec] = field(default_factory=list)
    reqs_to_store: list[ReqStoreSpec] = field(default_factory=list)


# =========================================================================================
# scheduler half
# =========================================================================================


class SchedulerHalf:
    def __init__(self, socket_path: str, block_tokens: int = 16, model_id: str = "default",
                 client: Optional[IPCClientSync] = None) -> None:
        self.block_tokens = block_tokens
        self.model_id = model_id
        self._ipc = client or IPCClientSync(socket_path)
        self._pending_loads: dict[str, list[ReqLoadSpec]] = {}
        self._pending_stores: dict[str, ReqStoreSpec] = {}
        self._pending_alloc: dict[str, dict[str, Any]] = {}
        self._stored: set[str] = set()
        self._negotiated = False
        self._compositions: "OrderedDict[str, int]" = OrderedDict()  # sightings of ordered chunk prefixes

    # -- prefix reuse (reference behaviour) -----------------------------------------------
    def get_num_new_matched_tokens(self, req_id: str, prompt_token_ids: Sequence[int],
                                   num_computed_tokens: int) -> tuple[int, bool]:
        """Tokens the connector can supply beyond ``num_computed_tokens`` (never asynchronous).

        One ``match_and_alloc`` round trip: a hit remembers the chunk to load, a miss
        remembers the server-side reservation to store into.  Repeated calls for the same
        request are harmless (the server returns the same reservation).
        """
        bt = self.block_tokens
        tokens = list(prompt_token_ids)
        aligned = (len(tokens) // bt) * bt
        if aligned == 0:
            return 0, False
        store_key = hash_tokens(tokens[:aligned])
        self._negotiate_once()
        t0 = time.perf_counter()
        try:
            with trace.span("rpc.match_and_alloc", "connector", req=req_id, tokens=len(tokens)):
                chunks, alloc = self._ipc.match_and_alloc(tokens, store_key, self.model_id)
        except RuntimeError as exc:
            logger.warning("[CONNECTOR] lookup failed for %s (%s): treating as a miss", req_id, exc)
            metrics.inc("connector.rpc_errors")
            return 0, False
        _perf.record("match_and_alloc_ms", (time.perf_counter() - t0) * 1e3, "ms")
        if chunks:
            best = chunks[0]
            usable = min(best["token_count"], aligned)
            # never claim the whole prompt: the engine must compute at least one token
            if usable >= len(tokens):
                usable = ((len(tokens) - 1) // bt) * bt
            extra = usable - num_computed_tokens
            if extra <= 0:
                return 0, False
            skip = num_computed_tokens // bt
            self._pending_loads[req_id] = [
                ReqLoadSpec(
                    chunk_key=best["chunk_key"], start_slot=best["start_slot"], num_slots=best["num_slots"],
                    block_ids=[], file_offset=best["file_offset"], token_count=usable,
                    pos_offset=best.get("pos_offset", 0), dst_token_offset=best.get("pos_offset", 0),
                    skip_slots=skip, req_id=req_id,
                )
            ]
            metrics.inc("connector.prefix_hits")
            return extra, False
        if alloc is not None:
            self._pending_alloc[req_id] = dict(alloc, first_block=hash_tokens(tokens[:bt]))
        metrics.inc("connector.prefix_misses")
        return 0, False

    # -- chunk reuse at arbitrary offsets ----------------------------------------------------
    def _negotiate_once(self) -> None:
        """First contact: packed token ids and the native lookup socket, if the server has them."""
        if not self._negotiated:
            if hasattr(self._ipc, "negotiate"):
                self._ipc.negotiate()
                # asked again at the next request if the server could not be reached this time
                self._negotiated = bool(getattr(self._ipc, "negotiated", True))
            else:
                self._negotiated = True

    def plan_chunk_loads(self, req_id: str, placements: Sequence[tuple[str, int]]) -> list[Optional[ReqLoadSpec]]:
        """Resolve ``(chunk_key, token offset)`` pairs; returns one spec (or None) per pair.

        Offsets must be block aligned.  Found chunks are queued for the request; the caller
        assigns their blocks with :meth:`assign_chunk_blocks`.
        """
        bt = self.block_tokens
        for _, off in placements:
            if off % bt:
                raise ValueError("chunk placements must be block aligned")
        self._negotiate_once()
        try:
            with trace.span("rpc.lookup_chunks", "connector", req=req_id, chunks=len(placements)):
                found = self._ipc.lookup_chunks([k for k, _ in placements], self.model_id)
        except RuntimeError as exc:
            logger.warning("[CONNECTOR] lookup_chunks failed for %s (%s)", req_id, exc)
            metrics.inc("connector.rpc_errors")
            found = [None] * len(placements)
        specs: list[Optional[ReqLoadSpec]] = []
        for (key, off), meta in zip(placements, found):
            if meta is None:
                metrics.inc("connector.chunk_misses")
                specs.append(None)
                continue
            metrics.inc("connector.chunk_hits")
            specs.append(
                ReqLoadSpec(
                    chunk_key=key, start_slot=meta["start_slot"], num_slots=meta["num_slots"], block_ids=[],
                    file_offset=meta["file_offset"], token_count=meta["token_count"],
                    pos_offset=meta.get("pos_offset", 0), dst_token_offset=off, req_id=req_id,
                )
            )
        self._pending_loads.setdefault(req_id, []).extend(s for s in specs if s is not None)
        return specs

    # -- composed chunks: the KV of an ordered combination, with its cross-attention --------------
    def composition_keys(self, chunks: Sequence[Sequence[int]]) -> list[str]:
        """Key of ``chunks[0] + ... + chunks[k]`` for every k (one streaming hash pass).  A
        combination is stored like any chunk, under the hash of its concatenated tokens: what
        makes it "composed" is that its KV was computed with the chunks attending to one another."""
        bt = self.block_tokens
        flat: list[int] = []
        ends = []
        for c in chunks:
            if len(c) % bt:
                raise ValueError("chunks must be a whole number of blocks")
            flat.extend(c)
            ends.append(len(flat) // bt)
        digests = prefix_digests(flat, bt)
        return [digests[e - 1] for e in ends]

    def merge_composed(self, chunks: Sequence[Sequence[int]]) -> list[list[int]]:
        """Replace the longest stored combination prefix ``chunks[:k]`` (k >= 2) by one chunk.

        The merged chunk sits at offset 0, so it is restored without re-rotation and is exact;
        the chunks after it are handled one by one as before.  One ``lookup_chunks`` round trip;
        on any error the list comes back unchanged."""
        chunks = [list(c) for c in chunks]
        if len(chunks) < 2:
            return chunks
        keys = self.composition_keys(chunks)
        try:
            found = self._ipc.lookup_chunks(keys[1:], self.model_id)
        except RuntimeError:
            return chunks
        for k in range(len(chunks), 1, -1):
            if found[k - 2] is not None:
                metrics.inc("connector.composed_hits")
                merged = [t for c in chunks[:k] for t in c]
                return [merged] + chunks[k:]
        return chunks

    def note_composition(self, chunks: Sequence[Sequence[int]], threshold: int, max_tracked: int = 4096) -> Optional[list[int]]:
        """Count sightings of the ordered pair-or-longer prefixes of ``chunks``; returns the
        concatenated tokens of the longest prefix that has now been seen ``threshold`` times and
        is not stored yet (the caller computes and stores it), else None."""
        if threshold <= 0 or len(chunks) < 2:
            return None
        keys = self.composition_keys(chunks)
        best = None
        for k in range(2, len(chunks) + 1):
            key = keys[k - 1]
            n = self._compositions.get(key, 0) + 1
            self._compositions[key] = n
            self._compositions.move_to_end(key)
            if n == threshold:
                best = k
        while len(self._compositions) > max_tracked:
            self._compositions.popitem(last=False)
        if best is None:
            return None
        return [t for c in chunks[:best] for t in c]

    def assign_chunk_blocks(self, req_id: str, request_block_ids: Sequence[int]) -> None:
        """Give every queued chunk load of ``req_id`` the request blocks its tokens fall into."""
        bt = self.block_tokens
        for spec in self._pending_loads.get(req_id, []):
            first = spec.dst_token_offset // bt + spec.skip_slots
            n = -(-spec.token_count // bt) - spec.skip_slots
            spec.block_ids = list(request_block_ids[first : first + n])

    def reserve_chunk_store(self, req_id: str, tokens: Sequence[int], block_ids: Sequence[int],
                            pos_offset: int = 0) -> Optional[ReqStoreSpec]:
        """Reserve slots for storing ``tokens`` (a whole number of blocks) keyed by their hash."""
        bt = self.block_tokens
        aligned = (len(tokens) // bt) * bt
        if aligned == 0:
            return None
        key = hash_tokens(list(tokens[:aligned]))
        try:
            a = self._ipc.alloc_chunk(key, aligned, self.model_id, pos_offset=pos_offset)
        except RuntimeError as exc:
            logger.info("[CONNECTOR] no reservation for %s: %s", key, exc)
            return None
        spec = ReqStoreSpec(
            chunk_key=key, start_slot=a["start_slot"], num_slots=a["num_slots"],
            block_ids=list(block_ids[: a["num_slots"]]), file_offset=a["file_offset"], token_count=aligned,
            pos_offset=pos_offset, first_block_digest=hash_tokens(list(tokens[:bt])), req_id=req_id,
        )
        self._pending_stores[req_id] = spec
        return spec

    # -- reference hooks -------------------------------------------------------------------------
    def update_state_after_alloc(self, req_id: str, block_ids: Sequence[int], num_external_tokens: int) -> None:
        bt = self.block_tokens
        loads = self._pending_loads.get(req_id)
        if loads and num_external_tokens > 0:
            spec = loads[0]
            first = spec.skip_slots
            n = -(-spec.token_count // bt) - first
            spec.block_ids = list(block_ids[first : first + n])
            return
        alloc = self._pending_alloc.pop(req_id, None)
        if alloc is not None:
            n = -(-alloc["token_count"] // bt)
            self._pending_stores[req_id] = ReqStoreSpec(
                chunk_key=alloc["chunk_key"], start_slot=alloc["start_slot"], num_slots=alloc["num_slots"],
                block_ids=list(block_ids[:n]), file_offset=alloc["file_offset"],
                token_count=alloc["token_count"], pos_offset=alloc.get("pos_offset", 0),
                first_block_digest=alloc.get("first_block", ""), req_id=req_id,
            )

    def build_connector_meta(self, scheduled_req_ids: Sequence[str]) -> ConnectorMeta:
        meta = ConnectorMeta()
        for req_id in scheduled_req_ids:
            loads = self._pending_loads.get(req_id)
            if loads and all(s.block_ids for s in loads):
                meta.reqs_to_load.extend(self._pending_loads.pop(req_id))
            store = self._pending_stores.get(req_id)
            if store is not None and store.block_ids:
                meta.reqs_to_store.append(self._pending_stores.pop(req_id))
                self._stored.add(store.chunk_key)
        if meta.reqs_to_load or meta.reqs_to_store:
            logger.debug("[CONNECTOR] step meta: %d loads, %d stores", len(meta.reqs_to_load),
                         len(meta.reqs_to_store))
        return meta

    def request_finished(self, req_id: str) -> tuple[bool, Optional[dict]]:
        self._pending_loads.pop(req_id, None)
        leftovers = [self._pending_alloc.pop(req_id, None), self._pending_stores.pop(req_id, None)]
        for item in leftovers:
            key = item["chunk_key"] if isinstance(item, dict) else getattr(item, "chunk_key", None)
            if key and key not in self._stored:
                try:
                    self._ipc.abort_chunk(key)
                except RuntimeError:
                    pass
        return False, None

    def close(self) -> None:
        self._ipc.close()


# =========================================================================================
# KV backends: how slot images get into and out of a paged pool
# =========================================================================================


class TorchKVBackend:
    """Pure-PyTorch restore/save on a ``[L, N, 2, H, B, D]`` pool (CPU engine and oracle)."""

    device_kind = "cpu"

    def __init__(self, geo: KVGeometry, pool_data: torch.Tensor, inv_freq: Sequence[float],
                 tp: int = 1, rank: int = 0) -> None:
        self.geo = geo
        self.pool = pool_data
        self.inv_freq = list(inv_freq)
        self.tp, self.rank = tp, rank
        self.h0, self.hn = tp_head_range(geo.num_kv_heads, tp, rank)

    def _split(self, images: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """uint8 ``[n, slot_size]`` -> float32 K, V ``[n, L, B, H, D]`` (all heads)."""
        g = self.geo
        n = images.shape[0]
        per_layer = images.reshape(n, g.num_layers, g.layer_size)
        shape = (n, g.num_layers, 2, g.block_tokens, g.num_kv_heads, g.head_dim)
        if g.codec == CODEC_FP8B16:
            pay = per_layer[..., : g.payload_bytes_per_layer].reshape(shape)
            sc = per_layer[..., g.payload_bytes_per_layer :].contiguous().view(torch.float32)
            kv = codec.dequantize_fp8b16(pay, sc.reshape(*shape[:-1], g.head_dim // 16))
        else:
            dt = {2: torch.bfloat16, 4: torch.float32}[g.dtype_bytes]
            kv = per_layer.contiguous().view(dt).reshape(shape).float()
        return kv[:, :, 0], kv[:, :, 1]

    def restore(self, images: torch.Tensor, block_ids: Sequence[int], deltas: Sequence[int]) -> None:
        if len(block_ids) == 0:
            return
        k, v = self._split(images.cpu())
        for i, d in enumerate(deltas):
            if d:
                k[i] = codec.rope_delta_rotate(k[i], int(d), self.inv_freq)
        sl = slice(self.h0, self.h0 + self.hn)
        idx = torch.as_tensor(list(block_ids), dtype=torch.long)
        # [n, L, B, H, D] -> pool [L, N, kv, H, B, D]
        self.pool[:, idx, 0] = k[..., sl, :].permute(1, 0, 3, 2, 4).to(self.pool.dtype).to(self.pool.device)
        self.pool[:, idx, 1] = v[..., sl, :].permute(1, 0, 3, 2, 4).to(self.pool.dtype).to(self.pool.device)

    def save(self, block_ids: Sequence[int], images: torch.Tensor) -> None:
        """Write this rank's head slice of each block into ``images`` (uint8 ``[n, slot_size]``)."""
        g = self.geo
        idx = torch.as_tensor(list(block_ids), dtype=torch.long)
        blk = self.pool[:, idx].cpu()  # [L, n, 2, H, B, D]
        for i in range(len(block_ids)):
            for layer in range(g.num_layers):
                k_new = blk[layer, i, 0].permute(1, 0, 2)  # [B, Hloc, D]
                v_new = blk[layer, i, 1].permute(1, 0, 2)
                region = images[i, layer * g.layer_size : (layer + 1) * g.layer_size]
                if self.tp == 1:
                    k_full, v_full = k_new, v_new
                else:
                    k_full, v_full = codec.unpack_layer(g, region, torch.float32)
                    k_full[:, self.h0 : self.h0 + self.hn] = k_new.float()
                    v_full[:, self.h0 : self.h0 + self.hn] = v_new.float()
                dt = {2: torch.bfloat16, 4: torch.float32}[g.dtype_bytes]
                region.copy_(codec.pack_layer(g, k_full.to(dt), v_full.to(dt)))


class CudaKVBackend:
    """Fused sm_100a restore/save kernels on a :class:`~daser_b200.ops.kv_ops.PagedKVPool`."""

    device_kind = "cuda"

    def __init__(self, geo: KVGeometry, pool, inv_freq: Sequence[float], max_pos: int = 8192,
                 rank: int = 0, max_slots: int = 4096, device: Optional[torch.device] = None) -> None:
        from daser_b200.ops import kv_ops

        self._ops = kv_ops
        self.geo, self.pool, self.rank = geo, pool, rank
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.cos_sin = kv_ops.rope_table(max_pos, inv_freq, self.device)
        self.status = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.max_slots = max_slots
        # persistent work-list buffers: pinned host mirror + device copy
        self._h = torch.empty((3, max_slots), dtype=torch.int64).pin_memory()
        self._d_ptr = torch.empty(max_slots, dtype=torch.int64, device=self.device)
        self._d_blk = torch.empty(max_slots, dtype=torch.int32, device=self.device)
        self._d_dlt = torch.empty(max_slots, dtype=torch.int32, device=self.device)
        self._uploaded: Optional[torch.cuda.Event] = None  # the mirror's last copy has been read
        self._consumed: Optional[torch.cuda.Event] = None  # the device list's last launch has run
        self.h2d_bytes = 0  # bytes of work lists copied to the device (callers read and reset it)

    def upload_worklist(self, ptrs: Sequence[int], block_ids: Sequence[int], deltas: Optional[Sequence[int]]):
        """Copy a work list to the device on the current stream; launches that use it follow on
        the same stream (or after an event recorded there)."""
        n = len(block_ids)
        if n > self.max_slots:
            raise ValueError(f"{n} slots in one step exceeds max_slots={self.max_slots}")
        for ev in (self._uploaded, self._consumed):
            if ev is not None:
                ev.synchronize()  # earlier copies / launches have read what is about to be overwritten
        h = self._h
        h[0, :n] = torch.as_tensor(list(ptrs), dtype=torch.int64)
        h[1, :n] = torch.as_tensor(list(block_ids), dtype=torch.int64)
        h[2, :n] = torch.as_tensor(list(deltas) if deltas is not None else [0] * n, dtype=torch.int64)
        self._d_ptr[:n].copy_(h[0, :n], non_blocking=True)
        self._d_blk[:n].copy_(h[1, :n], non_blocking=True)
        self._d_dlt[:n].copy_(h[2, :n], non_blocking=True)
        if self._uploaded is None:
            self._uploaded = torch.cuda.Event()
        self._uploaded.record()
        self.h2d_bytes += 24 * n
        return self._ops.KVWorkList(self._d_ptr[:n], self._d_blk[:n], self._d_dlt[:n] if deltas is not None else None)

    def _mark_consumed(self) -> None:
        if self._consumed is None:
            self._consumed = torch.cuda.Event()
        self._consumed.record()

    def restore_worklist(self, work, layer_begin: int = 0, layer_count: int = 0) -> None:
        """One launch over ``work`` for layers ``[layer_begin, layer_begin + layer_count)`` (0 = all)."""
        if work.n_slots:
            self._ops.kv_restore(work, self.geo, self.pool, self.cos_sin, self.status, layer_begin=layer_begin,
                                 layer_count=layer_count)
            self._mark_consumed()

    def restore_ptrs(self, ptrs: Sequence[int], block_ids: Sequence[int], deltas: Sequence[int]) -> None:
        if not block_ids:
            return
        self.restore_worklist(self.upload_worklist(ptrs, block_ids, deltas))

    def save_ptrs(self, ptrs: Sequence[int], block_ids: Sequence[int]) -> None:
        if not block_ids:
            return
        self._ops.kv_save(self.upload_worklist(ptrs, block_ids, None), self.geo, self.pool, self.rank, self.status)
        self._mark_consumed()

    def copy_rows(self, dst_ptr: int, src_ptr: int, pitch: int, width: int, rows: int) -> None:
        """``rows`` runs of ``width`` bytes, ``pitch`` apart on both sides, by the copy engine on the
        current stream (some layers of every slot image of a chunk, host tier to HBM tier)."""
        self._ops.copy_rows(dst_ptr, src_ptr, pitch, width, rows)
        self.h2d_bytes += width * rows

    def check_status(self) -> None:
        code, slot = self.status.tolist()
        if code:
            self.status.zero_()
            raise RuntimeError(f"KV kernel reported error {code} at work item {slot}")


# =========================================================================================
# worker half
# =========================================================================================


# a layer group's share of one slot image below which the chunk is read in one piece instead
MIN_STRIDED_READ = 128 << 10


@dataclass
class _LoadJob:
    """One chunk of a load: where the kernel reads it from and, if it is cold, where IO puts it."""

    spec: ReqLoadSpec
    n: int  # slots
    kind: str  # "hbm" | "host" | "host_fill" | "staging"
    src: int  # address of the first slot image the restore kernel reads
    io_dst: int = 0  # address the reads land at (0: no IO)
    promote_from: Optional[int] = None  # host address it is copied into the HBM tier from
    tickets: list = field(default_factory=list)  # one IO ticket per layer group


@dataclass
class LoadTicket:
    """A load in progress (see :meth:`WorkerHalf.begin_load`)."""

    jobs: list
    groups: list
    failed: set = field(default_factory=set)
    io_bytes: int = 0
    io_wait_ms: float = 0.0  # host time spent blocked on reads (what the pipeline could not hide)
    io_span_ms: float = 0.0  # first submit to last completion: the drive's view of the load
    t_submit: float = 0.0
    tier_bytes: dict = field(default_factory=dict)  # bytes restored by source: hbm / host / host_fill / staging
    work: Any = None
    waited: set = field(default_factory=set)  # (job, IO ticket) pairs already waited for


class WorkerHalf:
    """Moves KV between the store file, the optional HBM tier and the paged pool."""

    def __init__(self, socket_path: str, store_path: str, geo: KVGeometry, backend: Any,
                 io_backend: str = "auto", tp: int = 1, rank: int = 0, hbm_store: Any = None,
                 host_store: Any = None, client: Optional[IPCClientSync] = None, staging_slots: int = 256,
                 create_store_slots: int = 1024, commit: bool = True, write_behind: bool = False) -> None:
        from daser_b200.connector.transfer import TransferLayer

        # write_behind: `wait_for_save` returns once the blocks are copied into the staging arena
        # and their writes are submitted; the writes complete, and the chunks are committed, when
        # that half of the arena is needed again, before the next load that uses the arena, at
        # `flush_stores` or at shutdown.  The blocks may be reused at once either way; what changes
        # is the moment a chunk becomes visible to lookups.
        self._write_behind = bool(write_behind) and staging_slots >= 2
        self._pending_stores: dict = {}
        self._store_failed: set = set()
        self._next_half = 0

        self.geo = geo
        self.kv = backend
        self.tp, self.rank = tp, rank
        self.hbm = hbm_store
        self.host = host_store
        self._ipc = client or IPCClientSync(socket_path)
        self._commit = commit
        # geometry handshake: a store written with another slot size or codec must not be read
        try:
            self._ipc.hello({"slot_size": geo.slot_size, "block_tokens": geo.block_tokens})
        except RuntimeError as exc:
            if "geometry mismatch" in str(exc):
                raise ValueError(f"connector and control plane disagree: {exc}") from exc
            logger.warning("[CONNECTOR] geometry handshake skipped: %s", exc)
        if not os.path.exists(store_path):
            # the reference zero-fills max(slot_size * 1024, 64 MiB) through user space
            preallocate(store_path, max(geo.slot_size * create_store_slots, 64 << 20))
        is_cuda = backend.device_kind == "cuda"
        self._xfer = TransferLayer(store_path, backend=io_backend,
                                   device=torch.cuda.current_device() if is_cuda else None)
        # persistent staging: pinned host memory (readable by the kernels through UVA) for
        # host IO backends, device memory for GDS
        self._staging_slots = staging_slots
        nbytes = staging_slots * geo.slot_size
        if is_cuda and self._xfer.backend.name == "GDS":
            self._staging = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        elif is_cuda:
            self._staging = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        else:
            self._staging = torch.empty(nbytes, dtype=torch.uint8)
        # Plain host arenas the IO lands in are registered with the ring once (fixed-buffer IO: no
        # page pinning per read); a refusal (memlock limit) just leaves plain IO in place.
        # Arenas pinned by the CUDA driver are left alone: they are driver mappings, already
        # resident, and whether the kernel accepts them for long-term pinning differs by driver.
        regions = []
        for arena in (self._staging, host_store.arena if host_store is not None else None):
            if arena is not None and not arena.is_cuda and not arena.is_pinned():
                regions.append((arena.data_ptr(), arena.numel()))
        try:
            self.registered_regions = self._xfer.engine.register_buffers(regions)
        except (OSError, AttributeError):
            self.registered_regions = 0
        self._meta: Optional[ConnectorMeta] = None
        # (part, parts): this worker holds one of `parts` pieces of every chunk (per-rank store
        # files under vLLM tensor parallelism); the server publishes a chunk when all arrived
        self.commit_parts: Optional[tuple[int, int]] = None
        self._load_errors: set[int] = set()
        self._lock = threading.Lock()
        self.last_load_bytes = 0
        self.last_load_io_ms = 0.0
        self._load_done: Optional[Any] = None  # CUDA event: the last load's kernels have run

    @property
    def transfer(self):
        return self._xfer

    # -- metadata -------------------------------------------------------------------------------
    def bind_connector_metadata(self, meta: ConnectorMeta) -> None:
        self._meta = meta

    def clear_connector_metadata(self) -> None:
        self._meta = None

    # -- load -------------------------------------------------------------------------------------
    def start_load_kv(self) -> None:
        """Restore every chunk named by the bound metadata (synchronous with the step).

        Source of each chunk, first match wins: the HBM tier, the pinned host tier, the store
        file.  A cold chunk is read straight into slots reserved in the host tier when there
        is one (no staging copy), else into the staging arena.
        """
        meta = self._meta
        if meta is None or not meta.reqs_to_load:
            return
        with trace.span("start_load_kv", "connector", chunks=len(meta.reqs_to_load)):
            ticket = self.begin_load(meta)
            if ticket is not None:
                self.restore_group(ticket, 0)
                self.end_load(ticket, wait=True)

    def begin_load(self, meta: ConnectorMeta, layer_groups: Optional[Sequence[tuple[int, int]]] = None):
        """Start restoring ``meta.reqs_to_load``; returns a ticket, or None if there is nothing to do.

        ``layer_groups`` = ``[(first layer, count), ...]`` cuts the restore into pieces that
        :meth:`restore_group` finishes one by one, in order: the storage reads are issued here,
        all at once and group-major (every chunk's first layers come off the drive first), and
        piece ``g`` only waits for its own reads.  An engine launches the model's layers of
        group ``g`` right behind piece ``g``, so reading layers 10.. overlaps restoring and
        computing layers 0..9.  Without groups the whole chunk is one piece (one contiguous read).

        Chunks that do not fit the staging arena together are restored in waves; every wave
        but the last completes inside this call.
        """
        if meta is None or not meta.reqs_to_load:
            return None
        g = self.geo
        groups = [(int(a), int(n)) for a, n in (layer_groups or [(0, g.num_layers)])]
        if self.kv.device_kind != "cuda" and len(groups) != 1:
            raise ValueError("layer groups need the CUDA backend")
        waves: list[list[_LoadJob]] = [[]]
        used = 0
        for spec in meta.reqs_to_load:
            n = len(spec.block_ids)
            if n == 0:
                continue
            skip = spec.skip_slots * g.slot_size
            need = spec.skip_slots + n
            hit = self.hbm.lookup(spec.chunk_key, need) if self.hbm is not None else None
            if hit is not None:
                waves[-1].append(_LoadJob(spec, n, "hbm", hit + skip))
                continue
            hit = self.host.lookup(spec.chunk_key, need) if self.host is not None else None
            if hit is not None:
                waves[-1].append(_LoadJob(spec, n, "host", hit + skip))
                continue
            # only whole chunks enter a tier: a trimmed prefix hit (one slot short, so that the
            # engine has a token left to compute) must not be mistaken for the chunk later
            whole = spec.skip_slots == 0 and n == spec.num_slots
            if self.host is not None and whole:
                off = self.host.reserve(spec.chunk_key, n * g.slot_size)
                if off is not None:
                    ptr = self.host.arena.data_ptr() + off
                    waves[-1].append(_LoadJob(spec, n, "host_fill", ptr, io_dst=ptr))
                    continue
            # a chunk longer than the arena goes through it in pieces (each a run of its slots)
            cap = self._staging_slots
            pieces = [spec] if n <= cap else [
                dataclasses.replace(spec, block_ids=spec.block_ids[i:i + cap], skip_slots=spec.skip_slots + i)
                for i in range(0, n, cap)]
            for piece in pieces:
                m = len(piece.block_ids)
                if used + m > cap:
                    waves.append([])  # staging full: what we have goes first, to completion
                    used = 0
                ptr = self._staging.data_ptr() + used * g.slot_size
                waves[-1].append(_LoadJob(piece, m, "staging", ptr, io_dst=ptr))
                used += m
        self._wait_sources_free()
        for wave in waves[:-1]:
            t = self._issue(wave, [(0, g.num_layers)])
            self.restore_group(t, 0)
            self.end_load(t, wait=True, close_step=False)
        return self._issue(waves[-1], groups)

    def _wait_sources_free(self) -> None:
        """The previous load's kernels have read the staging arena (about to be refilled), and no
        store still writes from it."""
        self._complete_stores(None)
        if self._load_done is not None:
            self._load_done.synchronize()

    def _issue(self, jobs: list, groups: list[tuple[int, int]]) -> "LoadTicket":
        """Reserve HBM-tier room for what crosses PCIe, submit every read, upload the work list."""
        g = self.geo
        ticket = LoadTicket(jobs, groups)
        eng = self._xfer.engine
        cuda = self.kv.device_kind == "cuda"
        dev_staging = self._staging.is_cuda
        for job in jobs:
            spec = job.spec
            if job.kind != "hbm":
                metrics.inc("connector.bytes_over_pcie", job.n * g.slot_size)
                if cuda and self.hbm is not None and spec.skip_slots == 0 and job.n == spec.num_slots:
                    # Promote first, restore from the promoted copy: the images cross PCIe once,
                    # by DMA at full rate, instead of being read by the kernel and copied again.
                    off = self.hbm.reserve(spec.chunk_key, job.n * g.slot_size)
                    if off is not None:
                        job.promote_from, job.src = job.src, self.hbm.arena.data_ptr() + off
                if cuda and job.promote_from is None and not dev_staging:
                    self.kv.h2d_bytes += job.n * g.slot_size  # the kernel reads these images over PCIe itself
            ticket.tier_bytes[job.kind] = ticket.tier_bytes.get(job.kind, 0) + job.n * g.slot_size
        ticket.t_submit = time.perf_counter()
        whole = len(groups) == 1 and groups[0] == (0, g.num_layers)
        layer = g.layer_size
        # A group's share of one slot image is one read.  Where that is small (a small model's
        # slots), many short reads cost more than the overlap buys: the chunk is then read in one
        # piece, which the first group waits for and the others find done.
        if not whole and min(count for _, count in groups) * layer < MIN_STRIDED_READ:
            whole = True
        # reads go out group-major and, inside a group, in file order: neighbouring chunks
        # become one sequential sweep of the device
        for l0, count in ([(0, g.num_layers)] if whole else groups):
            for job in sorted((j for j in jobs if j.io_dst), key=lambda j: j.spec.file_offset):
                spec = job.spec
                off = spec.file_offset + spec.skip_slots * g.slot_size
                dev = dev_staging and job.kind == "staging"
                try:
                    if whole:
                        t = eng.submit_read(job.io_dst, off, job.n * g.slot_size, device=dev)
                    else:
                        t = eng.submit_read_strided(job.io_dst + l0 * layer, off + l0 * layer, count * layer, job.n,
                                                    g.slot_size, device=dev)
                except OSError as exc:
                    logger.warning("[CONNECTOR] read submit failed for %s: %s", spec.chunk_key, exc)
                    t = None
                job.tickets.extend([t] * (len(groups) if whole else 1))
                ticket.io_bytes += job.n * count * layer
        trace.instant("io.reads_submitted", n=sum(len(j.tickets) for j in jobs), bytes=ticket.io_bytes)
        if cuda:
            ticket.work = self._upload(ticket)
        return ticket

    def _upload(self, ticket: "LoadTicket"):
        g = self.geo
        ptrs: list[int] = []
        blocks: list[int] = []
        deltas: list[int] = []
        for job in ticket.jobs:
            if job.spec.chunk_key in ticket.failed:
                continue
            for i in range(job.n):
                ptrs.append(job.src + i * g.slot_size)
                blocks.append(job.spec.block_ids[i])
                deltas.append(job.spec.delta)
        return self.kv.upload_worklist(ptrs, blocks, deltas)

    def restore_group(self, ticket: "LoadTicket", index: int) -> None:
        """Finish piece ``index`` of the load: wait for its reads, then queue its copies into the
        HBM tier and its restore launch on the current stream.  Pieces are taken in order."""
        g = self.geo
        l0, count = ticket.groups[index]
        eng = self._xfer.engine
        t0 = time.perf_counter()
        newly_failed = False
        for job in ticket.jobs:
            if not job.io_dst or job.spec.chunk_key in ticket.failed:
                continue
            try:
                t = job.tickets[index]
                if t is None:
                    raise OSError("submit failed")
                if (id(job), t) in ticket.waited:
                    continue  # one read served several groups: an earlier group has waited for it
                ticket.waited.add((id(job), t))
                eng.wait(t)
            except (OSError, TimeoutError) as exc:
                logger.warning("[CONNECTOR] load of %s failed: %s", job.spec.chunk_key, exc)
                ticket.failed.add(job.spec.chunk_key)
                newly_failed = True
                for other in ticket.jobs:  # the same chunk may sit at several offsets of the request
                    if other.spec.chunk_key == job.spec.chunk_key:
                        self._load_errors.update(other.spec.block_ids)
                metrics.inc("connector.load_errors")
                # the reserved tier slots hold garbage
                if job.kind == "host_fill":
                    self.host.evict(job.spec.chunk_key)
                if job.promote_from is not None:
                    self.hbm.evict(job.spec.chunk_key)
                for later in job.tickets[index + 1:]:
                    try:  # its other reads still land in memory this step owns: let them finish
                        if later is not None and (id(job), later) not in ticket.waited:
                            ticket.waited.add((id(job), later))
                            eng.wait(later)
                    except (OSError, TimeoutError):
                        pass
        now = time.perf_counter()
        ticket.io_wait_ms += (now - t0) * 1e3
        if ticket.io_bytes and index + 1 == len(ticket.groups):
            ticket.io_span_ms = (now - ticket.t_submit) * 1e3
        if self.kv.device_kind != "cuda":
            jobs = [j for j in ticket.jobs if j.spec.chunk_key not in ticket.failed]
            images = torch.empty((sum(j.n for j in jobs), g.slot_size), dtype=torch.uint8)
            blocks: list[int] = []
            deltas: list[int] = []
            row = 0
            for job in jobs:
                for i in range(job.n):
                    images[row] = self._image_at(job.src + i * g.slot_size)
                    blocks.append(job.spec.block_ids[i])
                    deltas.append(job.spec.delta)
                    row += 1
            self.kv.restore(images, blocks, deltas)
            return
        if newly_failed:
            ticket.work = self._upload(ticket)  # without the failed chunk's slots
        layer = g.layer_size
        for job in ticket.jobs:
            if job.promote_from is not None and job.spec.chunk_key not in ticket.failed:
                self.kv.copy_rows(job.src + l0 * layer, job.promote_from + l0 * layer, g.slot_size, count * layer, job.n)
        whole = len(ticket.groups) == 1 and (l0, count) == (0, g.num_layers)
        self.kv.restore_worklist(ticket.work, 0 if whole else l0, 0 if whole else count)

    def reads_done(self, ticket: "LoadTicket") -> bool:
        """True once every storage read of the load has completed (nothing is waited for or consumed):
        an engine with other work, a decode batch, does that first while this is False."""
        eng = self._xfer.engine
        for job in ticket.jobs:
            for t in job.tickets:
                if t is not None and (id(job), t) not in ticket.waited and not eng.done(t):
                    return False
        return True

    def end_load(self, ticket: "LoadTicket", wait: bool = False, close_step: bool = True) -> None:
        """Every piece has been queued.  ``wait`` blocks until the kernels have run and raises on a
        kernel-reported error; without it the caller orders later work behind the current stream
        and checks :meth:`check_load_status` when it next synchronises anyway."""
        self.last_load_bytes, self.last_load_io_ms = ticket.io_bytes, ticket.io_wait_ms
        if ticket.io_bytes:
            _perf.record("load_io_ms", ticket.io_wait_ms, "ms")
            metrics.inc("connector.bytes_loaded", ticket.io_bytes)
        if self.kv.device_kind == "cuda":
            if self._load_done is None:
                self._load_done = torch.cuda.Event()
            self._load_done.record()
            if wait:
                self._load_done.synchronize()
                self.kv.check_status()
        if close_step:
            for tier in (self.hbm, self.host):
                if tier is not None:
                    tier.end_step()

    def check_load_status(self) -> None:
        if self.kv.device_kind == "cuda":
            self.kv.check_status()

    def _image_at(self, ptr: int) -> torch.Tensor:
        """CPU path: the slot image at host address ``ptr`` (staging or host tier)."""
        g = self.geo
        for arena in (self._staging, self.host.arena if self.host is not None else None):
            if arena is None or arena.is_cuda:
                continue
            base = arena.data_ptr()
            if base <= ptr < base + arena.numel():
                return arena[ptr - base : ptr - base + g.slot_size]
        raise ValueError("slot image address outside the host arenas")

    def wait_for_layer_load(self, layer_name: str) -> None:
        """Nothing to wait for: loads complete inside :meth:`start_load_kv`."""

    def take_load_errors(self) -> set[int]:
        """Block ids whose load failed since the last call (the engine recomputes them)."""
        out, self._load_errors = self._load_errors, set()
        return out

    # -- save --------------------------------------------------------------------------------------
    def save_kv_layer(self, layer_name: str, kv_layer: Any = None, attn_metadata: Any = None) -> None:
        """Nothing per layer: the blocks stay in the pool until :meth:`wait_for_save`, which
        gathers all layers with one launch."""

    def wait_for_save(self, barrier: Optional[Callable[[], None]] = None) -> None:
        meta = self._meta
        if meta is None or not meta.reqs_to_store:
            return
        with trace.span("wait_for_save", "connector", chunks=len(meta.reqs_to_store)):
            self._wait_for_save(meta, barrier)

    def _wait_for_save(self, meta: ConnectorMeta, barrier: Optional[Callable[[], None]]) -> None:
        """Pieces ``(spec, first staging slot, b0, b1)`` = blocks ``[b0, b1)`` of a chunk; as many as
        fit the staging arena (one half of it with ``write_behind``) go out together, and a longer
        chunk takes several rounds.  A chunk is committed once its last piece is on the drive and
        none failed."""
        halves = 2 if self._write_behind else 1
        cap = self._staging_slots // halves
        pending = [(spec, b0, min(b0 + cap, len(spec.block_ids)))
                   for spec in meta.reqs_to_store for b0 in range(0, len(spec.block_ids), cap)]
        failed = self._store_failed if self._write_behind else set()
        while pending:
            half = self._next_half if self._write_behind else 0
            self._complete_stores(half)  # the writes that still read this part of the arena
            batch, used = [], 0
            while pending and used + (pending[0][2] - pending[0][1]) <= cap:
                spec, b0, b1 = pending.pop(0)
                batch.append((spec, half * cap + used, b0, b1))
                used += b1 - b0
            tickets = self._store_batch(batch, barrier)
            if tickets is None:
                continue
            self._pending_stores[half] = (tickets, failed)
            if self._write_behind:
                self._next_half ^= 1  # returns with the writes in flight: the other half takes the next batch
            else:
                self._complete_stores(half)

    def _store_batch(self, batch, barrier):
        """Gather the batch's blocks into the arena (one launch) and submit its writes."""
        g = self.geo
        ptrs, blocks = [], []
        for spec, first, b0, b1 in batch:
            for i, b in enumerate(spec.block_ids[b0:b1]):
                ptrs.append(self._staging.data_ptr() + (first + i) * g.slot_size)
                blocks.append(b)
        if self.kv.device_kind == "cuda":
            self.kv.save_ptrs(ptrs, blocks)
            torch.cuda.current_stream().synchronize()  # images complete before the IO reads them
            self.kv.check_status()
        else:
            n = len(blocks)
            if n:
                first = batch[0][1]
                images = self._staging.view(-1, g.slot_size)[first : first + n]
                self.kv.save(blocks, images)
        if barrier is not None:
            barrier()  # every rank's head slice is in the owner's staging
        if not self._commit:
            return None
        eng = self._xfer.engine
        dev_staging = self._staging.is_cuda
        tickets = []
        for spec, first, b0, b1 in batch:
            ptr = self._staging.data_ptr() + first * g.slot_size
            tickets.append((spec, first, b0, b1, eng.submit_write(ptr, spec.file_offset + b0 * g.slot_size,
                                                                  (b1 - b0) * g.slot_size, device=dev_staging)))
        return tickets

    def _complete_stores(self, half: Optional[int] = None) -> None:
        """Finish the writes submitted from one half of the arena (all of it: ``None``): wait for
        them, hand whole chunks to the tiers, commit."""
        g = self.geo
        eng = self._xfer.engine
        for h in ([half] if half is not None else list(self._pending_stores)):
            entry = self._pending_stores.pop(h, None)
            if entry is None:
                continue
            tickets, failed = entry
            for spec, first, b0, b1, ticket in tickets:
                n = b1 - b0
                try:
                    eng.wait(ticket)
                except (OSError, TimeoutError) as exc:
                    logger.error("[CONNECTOR] store of %s failed: %s (reservation aborted)", spec.chunk_key, exc)
                    metrics.inc("connector.store_errors")
                    if spec.chunk_key not in failed:
                        failed.add(spec.chunk_key)
                        try:
                            self._ipc.abort_chunk(spec.chunk_key)
                        except RuntimeError:
                            pass
                    continue
                metrics.inc("connector.bytes_stored", n * g.slot_size)
                if b1 < len(spec.block_ids) or spec.chunk_key in failed:
                    continue  # more pieces to come, or an earlier piece was lost
                if b0 == 0:  # the whole chunk is in the arena: the tiers take it from there
                    if self.hbm is not None and self.kv.device_kind == "cuda":
                        self.hbm.admit(spec.chunk_key, self._staging, first * g.slot_size, n * g.slot_size)
                        self.hbm.end_step()
                    if self.host is not None:
                        self.host.admit(spec.chunk_key, self._staging, first * g.slot_size, n * g.slot_size)
                        self.host.end_step()
                try:
                    extra = {"first_block": spec.first_block_digest} if spec.first_block_digest else {}
                    if self.commit_parts is not None:
                        extra.update(part=self.commit_parts[0], parts=self.commit_parts[1])
                    self._ipc.commit_chunk(spec.chunk_key, **extra)
                except RuntimeError as exc:
                    logger.error("[CONNECTOR] commit of %s failed: %s", spec.chunk_key, exc)
        if not self._pending_stores:
            self._store_failed = set()

    def pending_store_keys(self) -> set:
        """Chunk keys whose writes are submitted but not yet committed (``write_behind``)."""
        return {t[0].chunk_key for tickets, _ in self._pending_stores.values() for t in tickets}

    def flush_stores(self) -> None:
        """With ``write_behind``: block until every submitted store is on the drive and committed."""
        self._complete_stores(None)

    def get_stats(self) -> dict[str, float]:
        return {k: v for k, v in metrics.snapshot().items() if k.startswith(("connector.", "transfer."))}

    def shutdown(self) -> None:
        try:
            try:
                self._complete_stores(None)
            except Exception as exc:  # noqa: BLE001
                logger.error("[CONNECTOR] pending stores lost at shutdown: %s", exc)
            self._xfer.close()
        finally:
            self._ipc.close()
