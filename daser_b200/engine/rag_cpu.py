"""CPU RAG engine: the toy decoder served through the connector with no GPU.

This is the minimum end-to-end slice: control plane, io_uring/file storage engine,
connector core, position re-encoding and a paged-KV decoder, all on CPU tensors.
Document chunks are prefilled stand-alone at positions ``0..n-1`` and stored; a request
``[prefix][chunk ...][query]`` restores each chunk at its new offset (keys rotated by the
offset) and only computes the prefix and the query.

The reference cannot do this: its service stores chunks keyed by their own hash but its
only lookup matches whole prompt prefixes, and nothing applies ``pos_offset``
(``daser/service/http_api.py:138-146``, ``daser/retrieval/prefix.py:63-72``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from daser_b200.connector.core import ConnectorMeta, SchedulerHalf, TorchKVBackend, WorkerHalf
from daser_b200.engine.request import RagRequest
from daser_b200.engine.scheduling import REJECT, START, SchedulingMixin
from daser_b200.hashing import hash_tokens
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import LlamaConfig, LlamaWeights, TorchPagedKV, reference_forward


@dataclass
class GenerateResult:
    generated: list[int]
    context_len: int
    restored_chunks: int
    finish_reason: str = "length"


class BlockAllocator:
    """Free-list allocator of pool blocks."""

    def __init__(self, num_blocks: int) -> None:
        self._free = list(range(num_blocks - 1, -1, -1))
        self.num_blocks = num_blocks

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise MemoryError(f"need {n} KV blocks, {len(self._free)} free")
        return [self._free.pop() for _ in range(n)]

    def free(self, blocks: Sequence[int]) -> None:
        self._free.extend(blocks)

    @property
    def num_free(self) -> int:
        return len(self._free)


@dataclass
class RequestResult:
    logits: torch.Tensor
    block_table: list[int]
    chunk_offsets: list[int]
    restored: list[bool]
    total_tokens: int


class CpuRagEngine(SchedulingMixin):
    # defaults of the optional behaviours, also for subclasses that build themselves differently
    compose_after = 0
    repair_tokens = 0

    def __init__(self, cfg: LlamaConfig, socket_path: str, store_path: str, num_blocks: int = 512,
                 codec_name: str = "raw", dtype: torch.dtype = torch.float32, seed: int = 0,
                 io_backend: str = "auto", model_id: str = "default", host_slots: int = 0,
                 compose_after: int = 0, repair_tokens: int = 0, weights: Optional[LlamaWeights] = None) -> None:
        self.cfg = cfg
        # > 0: after a chunk was restored behind other context, its first `repair_tokens` tokens are
        # recomputed in place with attention over everything before them (the tokens whose stored KV
        # is furthest from what the full context would have produced: they saw nothing when stored)
        self.repair_tokens = repair_tokens
        # > 0: an ordered combination of chunks seen this many times is computed once with full
        # cross-attention and stored; later requests that start with it restore it as one chunk
        self.compose_after = compose_after
        self.weights = weights if weights is not None else LlamaWeights.random(cfg, "cpu", dtype, seed=seed)
        self.pool = TorchPagedKV(cfg, num_blocks, dtype)
        self.blocks = BlockAllocator(num_blocks)
        self.geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens,
                              {torch.float32: 4, torch.bfloat16: 2}[dtype], codec_name)
        self.sched = SchedulerHalf(socket_path, cfg.block_tokens, model_id)
        from daser_b200.kv.hbm_store import HBMStore

        self.host = HBMStore(self.geo.slot_size, host_slots, torch.device("cpu")) if host_slots > 0 else None
        self.worker = WorkerHalf(socket_path, store_path, self.geo,
                                 TorchKVBackend(self.geo, self.pool.data, cfg.inv_freq()), io_backend=io_backend,
                                 host_store=self.host)
        self._req = 0
        self.waiting: list[RagRequest] = []
        self.running: list[RagRequest] = []

    # -- hooks a multi-process arrangement overrides (pipeline stages: parallel/pp.py) ------------
    def _lead(self, fn):
        """Run ``fn`` where the scheduler half lives; every process gets its result."""
        return fn()

    def _forward(self, tokens: Sequence[int], positions: torch.Tensor, table: torch.Tensor, context_len: int,
                 return_logits: bool = True) -> Optional[torch.Tensor]:
        return reference_forward(self.weights, torch.tensor(list(tokens)), positions, self.pool, table, context_len,
                                 return_logits=return_logits)

    def _sample(self, logits: Optional[torch.Tensor], req: Optional[RagRequest] = None) -> int:
        """Greedy, or (request with a temperature) a draw from softmax(logits / T) by the Gumbel-max
        rule, reproducible from the request's seed and the step."""
        row = logits[-1].float()
        if req is not None and req.truncated():
            from daser_b200.engine.sampling import apply_truncation

            row = row.clone()[None]
            apply_truncation(row, torch.tensor([1.0 / req.temperature]), torch.tensor([req.top_k]),
                             torch.tensor([req.top_p]))
            row = row[0]
        if req is not None and req.temperature > 0:
            gen = torch.Generator().manual_seed(req.step_seed())
            u = torch.rand(row.shape, generator=gen).clamp_(1e-9, 1.0 - 1e-9)
            row = row / req.temperature - torch.log(-torch.log(u))
        return int(row.argmax())

    def _next_id(self) -> str:
        self._req += 1
        return f"req-{self._req}"

    def _step(self, meta: ConnectorMeta, fn):
        self.worker.bind_connector_metadata(meta)
        try:
            self.worker.start_load_kv()
            out = fn()
            self.worker.wait_for_save()
        finally:
            self.worker.clear_connector_metadata()
        return out

    # -- offline: fill the chunk store -----------------------------------------------------
    def store_chunk(self, tokens: Sequence[int]) -> str:
        """Prefill ``tokens`` alone at positions 0.. and store their KV; returns the chunk key."""
        bt = self.cfg.block_tokens
        tokens = list(tokens)
        if len(tokens) % bt:
            raise ValueError("chunks must be a whole number of blocks")
        req = self._next_id()
        table = self.blocks.alloc(len(tokens) // bt)

        def plan():
            spec = self.sched.reserve_chunk_store(req, tokens, table, pos_offset=0)
            return self.sched.build_connector_meta([req]) if spec is not None else ConnectorMeta()

        meta = self._lead(plan)
        self._step(meta, lambda: self._forward(tokens, torch.arange(len(tokens)), torch.tensor(table), 0,
                                               return_logits=False))
        self._lead(lambda: self.sched.request_finished(req))
        self.blocks.free(table)
        return hash_tokens(tokens)

    # -- online: a RAG request -----------------------------------------------------------------
    def run_request(self, prefix: Sequence[int], chunks: Sequence[Sequence[int]], query: Sequence[int],
                    keep_blocks: bool = False) -> RequestResult:
        bt = self.cfg.block_tokens
        if len(prefix) % bt:
            raise ValueError("the prefix must end on a block boundary")
        req = self._next_id()
        offsets, pos = [], len(prefix)
        for c in chunks:
            if len(c) % bt:
                raise ValueError("chunks must be a whole number of blocks")
            offsets.append(pos)
            pos += len(c)
        total = pos + len(query)
        table = self.blocks.alloc(-(-total // bt))
        tbl = torch.tensor(table)
        placements = [(hash_tokens(list(c)), off) for c, off in zip(chunks, offsets)]

        def plan():
            found = self.sched.plan_chunk_loads(req, placements)
            self.sched.assign_chunk_blocks(req, table)
            return found, self.sched.build_connector_meta([req])

        specs, meta = self._lead(plan)

        def run():
            # the prefix is computed, then every chunk that could not be restored, then the query
            ctx = 0
            if prefix:
                self._forward(prefix, torch.arange(len(prefix)), tbl, 0, return_logits=False)
            ctx = len(prefix)
            for c, off, spec in zip(chunks, offsets, specs):
                if spec is None:
                    self._forward(c, torch.arange(off, off + len(c)), tbl, ctx, return_logits=False)
                elif self.repair_tokens > 0 and off > 0:
                    r = min(self.repair_tokens, len(c))
                    self._forward(c[:r], torch.arange(off, off + r), tbl, off, return_logits=False)
                ctx = off + len(c)
            return self._forward(query, torch.arange(ctx, ctx + len(query)), tbl, ctx)

        logits = self._step(meta, run)
        self._lead(lambda: self.sched.request_finished(req))
        if not keep_blocks:
            self.blocks.free(table)
        return RequestResult(logits, table, offsets, [s is not None for s in specs], total)

    def generate(self, chunks: Sequence[Sequence[int]], query: Sequence[int], max_new_tokens: int = 1,
                 store_misses: bool = False, on_token=None, temperature: float = 0.0,
                 seed: int = 0, stop_token_ids: Sequence[int] = (), top_k: int = 0,
                 top_p: float = 1.0) -> "GenerateResult":
        """Serve one request to completion with greedy sampling: the same call the GPU engine
        offers (``GpuRagEngine.generate``), on the oracle model.  ``store_misses`` is accepted
        for signature parity; chunks are only stored through :meth:`store_chunk` here.
        ``on_token(token_id)`` is called as each token is sampled (streaming front ends)."""
        req = self.submit(RagRequest([list(c) for c in chunks], list(query), max_new_tokens,
                                     temperature=float(temperature), seed=int(seed), top_k=int(top_k),
                                     top_p=float(top_p), stop_token_ids=tuple(int(t) for t in stop_token_ids)))
        sent = 0
        while not req.done:
            self.step()
            if on_token is not None:
                for tok in req.generated[sent:]:
                    on_token(tok)
                sent = len(req.generated)
        if req.error is not None:
            raise MemoryError(req.error)
        return GenerateResult(req.generated, req.context_len, req.restored_chunks, req.finish_reason)

    # -- iteration-level scheduling: the calls GpuRagEngine offers, on the oracle model ----------
    def submit(self, req: RagRequest) -> RagRequest:
        req.req_id = req.req_id or self._next_id()
        if self.compose_after > 0 and not req.asked:
            req.asked = [list(c) for c in req.chunks]
            req.chunks = self._lead(lambda: self.sched.merge_composed(req.asked))
        self.waiting.append(req)
        return req

    def _after_finish(self, req: RagRequest) -> None:
        """Between two steps, once a request has ended: a chunk combination seen often enough is
        computed from scratch (its chunks attending to one another) and stored whole."""
        room = sum(len(c) for c in req.asked) // self.cfg.block_tokens <= self.blocks.num_free
        if self.compose_after > 0 and req.asked and req.error is None and room:  # (no room: next sighting)
            combo = self._lead(lambda: self.sched.note_composition(req.asked, self.compose_after))
            if combo is not None:
                self.store_chunk(combo)

    def step(self) -> None:
        """One engine iteration: the prefill of the oldest waiting request (restore, compute
        what is missing, first token), else one more token for every running request."""
        bt = self.cfg.block_tokens
        decision = self._admission() if self.waiting else None
        if decision == REJECT:
            return
        if decision == START:
            req = self.waiting.pop(0)
            res = self.run_request([], req.chunks, req.query, keep_blocks=True)
            req.block_table, req.context_len = list(res.block_table), res.total_tokens
            req.block_table.extend(self.blocks.alloc(req.blocks_needed(bt) - len(req.block_table)))
            req.restored_chunks = sum(res.restored)
            req.generated.append(self._sample(res.logits, req))
            self.running.append(req)
        else:
            for req in list(self.running):
                pos = req.context_len + len(req.generated) - 1
                logits = self._forward([req.generated[-1]], torch.tensor([pos]), torch.tensor(req.block_table), pos)
                req.generated.append(self._sample(logits, req))
        for req in list(self.running):
            if req.finished():
                req.done = True
                self.running.remove(req)
                self.blocks.free(req.block_table)
                self._after_finish(req)

    def recompute_chunk_alone(self, chunk: Sequence[int], offset: int) -> tuple[list[int], int]:
        """Run ``chunk`` alone at positions ``offset..``; returns its (fresh) blocks and length.

        RoPE attention depends only on position differences, so the hidden states, the values
        and the un-rotated keys equal those of the stand-alone prefill at 0: the restored,
        re-rotated KV must match this recomputation.
        """
        bt = self.cfg.block_tokens
        table = self.blocks.alloc(len(chunk) // bt)
        self._forward(chunk, torch.arange(offset, offset + len(chunk)), torch.tensor(table), 0, return_logits=False)
        return table, len(chunk)

    def close(self) -> None:
        self.worker.shutdown()
        self.sched.close()
