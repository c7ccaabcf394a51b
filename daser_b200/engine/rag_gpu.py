"""GPU RAG engine: the native serving engine behind the service and the benchmarks.

The reference relies on a separately launched ``vllm serve`` for this part
(``daser/service/vllm_client.py``); here the engine is in-process.  It combines

* :class:`~daser_b200.engine.runner.GpuModelRunner` (model forward on the sm_100a kernels),
* the connector halves (:mod:`daser_b200.connector.core`) with the fused restore / save
  kernels, the native storage engine and the optional HBM tier,
* an iteration-level scheduler: a waiting request is admitted with one *TTFT step*
  (look up its chunks, restore them at their new offsets, prefill whatever was not cached
  plus the query, sample the first token); otherwise all running sequences decode one token
  as a batch.

A TTFT step is pipelined by layer group (``GpuModelRunner.layer_groups``): the storage reads of
every cold chunk are issued at once, group-major; restore piece ``g`` (its copies into the HBM
tier and its fused kernel) runs on a side stream as soon as the reads of its layers are in, and
the model's layers of group ``g`` are launched behind it.  Reading layers 10.. from the drive
overlaps restoring and computing layers 0..9, and a step whose chunks are all in memory tiers
waits for the first piece only.

With ``tp > 1`` every rank runs the same engine object in lock step.  Rank 0 owns the scheduler
half and publishes each step's plan through a shared-memory mailbox.  Every rank owns the
chunks whose key hashes to it: it keeps them in its own HBM and host tiers, reads them from the
store with its own IO ring over its own PCIe link, and its restore kernel scatters each head
slice into every rank's paged pool over NVLink; a per-source flag per layer group, written
behind the kernel and awaited (bounded) in front of each rank's layers, replaces a barrier.
"""

from __future__ import annotations

import contextlib
import os
import time
from typing import Optional, Sequence

import torch

from daser_b200 import metrics
from daser_b200.connector.core import ConnectorMeta, CudaKVBackend, SchedulerHalf, WorkerHalf
from daser_b200.engine.rag_cpu import BlockAllocator
from daser_b200.engine.request import RagRequest
from daser_b200.engine.scheduling import REJECT, START, SchedulingMixin
from daser_b200.engine.runner import GpuModelRunner
from daser_b200.hashing import hash_tokens
from daser_b200.kv.hbm_store import HBMStore
from daser_b200.models.llama import LlamaConfig, LlamaWeights
from daser_b200.ops import gemm as gemm_ops
from daser_b200.utils import trace


class GpuRagEngine(SchedulingMixin):
    def __init__(self, cfg: LlamaConfig, socket_path: str, store_path: str, num_blocks: int = 4096,
                 max_tokens: int = 256, max_seqs: int = 64, hbm_slots: int = 0, host_slots: int = 0,
                 io_backend: str = "auto",
                 seed: int = 0, model_id: str = "default", tp_ctx=None, weights: Optional[LlamaWeights] = None,
                 staging_slots: int = 512, max_blocks: int = 512, use_graphs: bool = True,
                 compose_after: int = 0, repair_tokens: int = 0, layer_groups: int = 8, pp_link=None,
                 write_behind: bool = False) -> None:
        self.cfg = cfg
        # pipeline parallelism: this process is one stage (``parallel/pp.py::StageLink``); it runs a
        # contiguous range of layers, keeps their KV in a pool and a store file of its own, and a
        # chunk is published once every stage has committed its part
        self.pp_link = pp_link
        if pp_link is not None and tp_ctx is not None:
            raise ValueError("pipeline stages are single-GPU here: pass tp_ctx or pp_link, not both")
        # > 0: after a chunk was restored behind other context, its first `repair_tokens` tokens are
        # recomputed in place with attention over everything before them (the tokens whose stored KV
        # is furthest from what the full context would have produced: they saw nothing when stored)
        self.repair_tokens = repair_tokens
        # > 0: an ordered combination of chunks seen this many times is computed once with full
        # cross-attention and stored; later requests that start with it restore it as one chunk
        self.compose_after = compose_after
        self.tp = tp_ctx.tp if tp_ctx is not None else 1
        self.rank = tp_ctx.rank if tp_ctx is not None else 0
        self.tp_ctx = tp_ctx
        self.device = torch.device("cuda", torch.cuda.current_device())
        layer_range, pool_layers = None, None
        if pp_link is not None:
            from daser_b200.parallel.pp import partition_layers, stage_store_path

            layer_range = partition_layers(cfg.num_layers, pp_link.stages)[pp_link.stage]
            pool_layers = max(len(r) for r in partition_layers(cfg.num_layers, pp_link.stages))
            store_path = stage_store_path(store_path, pp_link.stage, pp_link.stages)
        self.weights = weights or LlamaWeights.random(cfg, self.device, torch.bfloat16, tp=self.tp,
                                                      rank=self.rank, seed=seed, layers=layer_range)
        # the engine owns its weights: put gate/up rows in the order that lets SwiGLU run as the
        # GEMM's epilogue (in place, one layer-sized temporary)
        if self.weights.gate_up_block == 0 and self.weights.inter_local % gemm_ops.GATE_UP_BLOCK == 0:
            self.weights.interleave_gate_up_(gemm_ops.GATE_UP_BLOCK)
        self.runner = GpuModelRunner(cfg, self.weights, num_blocks, max_tokens, max_seqs, tp_ctx, self.device,
                                     max_blocks=max_blocks, use_graphs=use_graphs, layer_groups=layer_groups,
                                     layer_range=layer_range, pool_layers=pool_layers, pp_link=pp_link)
        self.blocks = BlockAllocator(num_blocks)
        self.max_blocks_per_seq = max_blocks  # the runner's block tables are this wide
        self.geo = self.runner.geo
        # the restore kernel of the IO owner scatters into every rank's pool
        pool = tp_ctx.global_pool(self.runner) if tp_ctx is not None else self.runner.local_pool
        self.kv_backend = CudaKVBackend(self.geo, pool, cfg.inv_freq(), max_pos=self.runner.cos_sin.shape[0],
                                        rank=self.rank, max_slots=max(staging_slots, 1024), device=self.device)
        self.kv_backend.cos_sin = self.runner.cos_sin
        # tiers and IO are per rank: `hbm_slots` / `host_slots` are this rank's share
        # Opt-in: decode batches run inside a starting request's wait for the drive (not with
        # composed-chunk stores, which a finishing request would start inside that wait).  Measured on
        # the saturated one-GPU open loop (4 req/s x 128 tokens of a 70B model): output 366 -> 388 tok/s
        # and TTFT p99 1953 -> 780 ms, but TTFT p50 187 -> 321 ms; prefill-first stays the default.
        self.interleave_decode = os.environ.get("DASER_INTERLEAVE_DECODE", "0") == "1" and compose_after == 0
        self.hbm = HBMStore(self.geo.slot_size, hbm_slots, self.device) if hbm_slots > 0 else None
        self.host = HBMStore(self.geo.slot_size, host_slots, torch.device("cpu")) if host_slots > 0 else None
        self.is_lead = self.rank == 0 and (pp_link is None or pp_link.first)  # plans, reserves, finishes
        self.sched = SchedulerHalf(socket_path, cfg.block_tokens, model_id) if self.is_lead else None
        if self.tp > 1 and self.rank != 0:
            tp_ctx.wait_for_path(store_path)  # rank 0 creates the store file
        self.worker = WorkerHalf(socket_path, store_path, self.geo, self.kv_backend, io_backend=io_backend, tp=self.tp,
                                 rank=self.rank, hbm_store=self.hbm, host_store=self.host, staging_slots=staging_slots,
                                 write_behind=write_behind and self.tp == 1 and pp_link is None)
        if pp_link is not None and pp_link.stages > 1:
            self.worker.commit_parts = (pp_link.stage, pp_link.stages)
        # Every process has now shaken hands with the control plane, which may live on a thread of
        # the lead process.  Meet here before anyone goes on: collective set-up calls (symmetric
        # memory rendezvous, communicator creation) can block without releasing the interpreter
        # lock, and a lead that enters one while a peer still waits for the control plane's answer
        # would starve the very thread that has to give it.
        if tp_ctx is not None:
            tp_ctx.barrier()  # (releases the lock while it waits: the control plane keeps answering)
            tp_ctx.prepare_save_staging(self.geo)  # a rendezvous: only now, with every rank at this line
        elif pp_link is not None:
            pp_link.barrier()
        self.waiting: list[RagRequest] = []
        self.running: list[RagRequest] = []
        self._n = 0
        self._ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        self._restore_stream = torch.cuda.Stream(device=self.device)
        self._group_ev = [torch.cuda.Event() for _ in self.runner.layer_groups]
        self._kv_epoch = 0  # restore pieces signalled so far (the same on every rank)
        self.h2d_bytes = 0  # host -> device bytes of the steps so far (inputs, work lists, tier promotions)

    # ------------------------------------------------------------------------------------------
    def _next_id(self) -> str:
        self._n += 1
        return f"r{self._n}"

    def _sync_ranks(self) -> None:
        if self.tp_ctx is not None:
            self.tp_ctx.barrier()

    def _bcast(self, obj):
        """``obj`` of the lead process (tensor-parallel rank 0 / pipeline stage 0) everywhere."""
        if self.tp_ctx is not None:
            return self.tp_ctx.broadcast_object(obj)
        if self.pp_link is not None:
            return self.pp_link.from_stage(obj, 0)
        return obj

    def _tokens_out(self, sampled: Optional[torch.Tensor], n: int) -> list[int]:
        """The step's sampled tokens on the host (read back from the device; in a pipeline, sent
        from the last stage to every stage)."""
        if self.pp_link is None:
            return [int(t) for t in sampled[:n].tolist()]
        return self.pp_link.tokens_from_last(sampled[:n] if sampled is not None else None, n, self.device)

    def owner_of(self, chunk_key: str) -> int:
        """The rank that keeps ``chunk_key`` in its tiers and moves it between the store and the pools."""
        return int(chunk_key[:8], 16) % self.tp if self.tp > 1 else 0

    def _prefill_tokens(self, tokens: Sequence[int], start_pos: int, table: list[int],
                        sample: Optional[dict] = None, gate=None) -> torch.Tensor:
        """Run ``tokens`` through the model in pieces of at most ``max_tokens``; returns the last sample
        (greedy, or drawn with ``sample = {"temperature", "seed"}``).  ``gate`` (see
        ``GpuModelRunner.forward``) applies to the first piece."""
        out = None
        mt = self.runner.max_tokens
        for i in range(0, len(tokens), mt):
            piece = list(tokens[i : i + mt])
            inp = self.runner.stage_inputs([{"tokens": piece, "start_pos": start_pos + i, "block_table": table,
                                             **(sample or {})}])
            self.h2d_bytes += self.runner.h2d_bytes
            out = self.runner.forward(inp, gate=gate if i == 0 else None)
        return out

    def warm_up(self, token_counts: Sequence[int] = (64,), context_lens: Sequence[int] = (2048, 4096, 8192),
                decode_batches: Sequence[int] = ()) -> None:
        """Run (and capture) the forward for the step shapes a workload will use, on scratch blocks.

        A shape's first run is eager and its second run captures a CUDA graph, which costs
        tens of milliseconds; serving code calls this once at start-up so that no request pays it.
        ``token_counts`` are single-sequence prefill steps, ``decode_batches`` decode steps of that
        many sequences (see :meth:`decode_bucket`), each at every context length.
        """
        bt = self.cfg.block_tokens
        for ctx in context_lens:
            n_blocks = -(-ctx // bt)
            if n_blocks > self.blocks.num_free or n_blocks > self.runner.max_blocks:
                continue
            table = self.blocks.alloc(n_blocks)
            shapes = [[{"tokens": [1] * t, "start_pos": ctx - t, "block_table": table}]
                      for t in token_counts if t <= self.runner.max_tokens]
            shapes += [[{"tokens": [1], "start_pos": ctx - 1, "block_table": table}] * b
                       for b in decode_batches if b <= self.runner.max_seqs]
            for seqs in shapes:
                for _ in range(3):
                    self.runner.forward(self.runner.stage_inputs(seqs))
                torch.cuda.synchronize()
            self.blocks.free(table)

    # -- offline fill ------------------------------------------------------------------------------
    def store_chunk(self, tokens: Sequence[int]) -> str:
        """Prefill ``tokens`` alone at positions 0.. and write their KV to the store."""
        bt = self.cfg.block_tokens
        tokens = list(tokens)
        if len(tokens) % bt:
            raise ValueError("chunks must be a whole number of blocks")
        table = self.blocks.alloc(len(tokens) // bt)
        req = self._next_id()
        meta = ConnectorMeta()
        if self.sched is not None:
            if self.sched.reserve_chunk_store(req, tokens, table, pos_offset=0) is not None:
                meta = self.sched.build_connector_meta([req])
        meta = self._bcast(meta)
        self._prefill_tokens(tokens, 0, table)
        self._save(meta)
        self.worker.flush_stores()  # an explicit store is visible when this returns
        if self.pp_link is not None:
            self.pp_link.barrier()  # every stage has committed its part: the chunk is visible when this returns
        if self.sched is not None:
            self.sched.request_finished(req)
        self.blocks.free(table)
        return hash_tokens(tokens)

    def _save(self, meta: ConnectorMeta) -> None:
        if self.tp_ctx is None:
            self.worker.bind_connector_metadata(meta)
            try:
                self.worker.wait_for_save()
            finally:
                self.worker.clear_connector_metadata()
            return
        self.tp_ctx.save_step(self, meta)

    def _begin_restore(self, meta: ConnectorMeta):
        """Issue this rank's share of the step's loads; returns ``(ticket, gate)`` for the first
        forward of the step (``gate`` is None when no rank restores anything)."""
        loads = list(meta.reqs_to_load)
        if not loads:
            return None, None
        mine = ConnectorMeta(reqs_to_load=[s for s in loads if self.owner_of(s.chunk_key) == self.rank])
        # the worker counts layers inside a slot image: from 0 in every pipeline stage
        groups = [(a - self.runner.layers.start, n) for a, n in self.runner.layer_groups]
        ticket = self.worker.begin_load(mine, groups) if mine.reqs_to_load else None
        side = self._restore_stream
        base = self._kv_epoch
        self._kv_epoch += len(groups)
        tp = self.tp_ctx

        def on_side():
            return torch.cuda.stream(side) if side is not None else contextlib.nullcontext()

        def gate(g: int) -> None:
            # piece g: wait for its reads (host), queue its copies and kernel on the side stream
            with on_side():
                if ticket is not None:
                    self.worker.restore_group(ticket, g)
                if tp is not None:
                    tp.signal_kv_landed(base + g + 1)  # behind this rank's scatter into every pool
                if side is not None:
                    self._group_ev[g].record(side)
            if side is not None:
                torch.cuda.current_stream().wait_event(self._group_ev[g])
            if tp is not None:
                tp.wait_kv_landed(base + g + 1, self.runner.status)  # every rank's piece g is in this pool
            if g + 1 == len(groups) and ticket is not None:
                with on_side():
                    self.worker.end_load(ticket)

        return ticket, gate

    # -- online ---------------------------------------------------------------------------------------
    def submit(self, req: RagRequest) -> RagRequest:
        req.req_id = req.req_id or self._next_id()
        req.arrival = req.arrival or time.perf_counter()
        if self.compose_after > 0 and not req.asked:
            # the rank that owns the scheduler half decides; every rank must serve the same list
            req.asked = [list(c) for c in req.chunks]
            req.chunks = self._bcast(self.sched.merge_composed(req.asked) if self.sched is not None else None)
        self.waiting.append(req)
        return req

    def step(self) -> None:
        if self.tp_ctx is not None:
            self.tp_ctx.check_peers()  # host-side: a lost peer ends the step before any launch
        decision = self._admission() if self.waiting else None
        if decision == REJECT:
            return
        if decision == START:
            with trace.span("engine.ttft_step", "engine"):
                self._ttft_step(self.waiting.pop(0))
        elif self.running:  # nothing waiting, or the head of the queue waits for blocks
            with trace.span("engine.decode_step", "engine", batch=len(self.running)):
                self._decode_step()

    def _ttft_step(self, req: RagRequest) -> None:
        cfg, bt = self.cfg, self.cfg.block_tokens
        t_start = time.perf_counter()
        self._ev[0].record()
        h2d0 = self.h2d_bytes + self.kv_backend.h2d_bytes
        offsets, pos = [], 0
        for c in req.chunks:
            if len(c) % bt:
                raise ValueError("chunks must be a whole number of blocks")
            offsets.append(pos)
            pos += len(c)
        total = pos + len(req.query)
        n_blocks = -(-(total + req.max_new_tokens) // bt)
        req.block_table = self.blocks.alloc(n_blocks)
        # 1. plan: which chunks are cached, where do they go
        plan = None
        if self.sched is not None:
            placements = [(hash_tokens(c), off) for c, off in zip(req.chunks, offsets)]
            if self.worker.pending_store_keys() & {k for k, _ in placements}:
                self.worker.flush_stores()  # a chunk this request asks for is still on its way to the drive
            specs = self.sched.plan_chunk_loads(req.req_id, placements)
            self.sched.assign_chunk_blocks(req.req_id, req.block_table)
            plan = (self.sched.build_connector_meta([req.req_id]), [s is not None for s in specs])
        meta, found = self._bcast(plan)
        t_plan = time.perf_counter()
        # 2. start restoring the cached chunks: reads go out now, the pieces follow group by group
        #    in front of the first forward below
        self._ev[1].record()
        ticket, gate = self._begin_restore(meta)
        t_restore = time.perf_counter()
        # While this request's chunks are still coming off the drive, the requests that are already
        # decoding go on: a decode batch per look at the reads (every rank takes the same decision).
        while self.interleave_decode and self.running and meta.reqs_to_load and self.pp_link is None:
            done = ticket is None or self.worker.reads_done(ticket)
            if self.tp_ctx is not None:
                done = all(self.tp_ctx.gather_object(bool(done)))
            if done:
                break
            self._decode_step()
        sample = ({"temperature": req.temperature, "seed": req.step_seed(), "top_k": req.top_k, "top_p": req.top_p}
                  if req.temperature > 0 else None)

        def compute(failed_blocks: set, gate) -> torch.Tensor:
            """Prefill whatever is not (validly) restored, then the query; returns the sampled token.
            Neighbouring pieces that must be computed (missed chunks, and the query behind them) go
            through the model as ONE run of tokens: every forward streams all the weights, so a
            request whose chunks all miss costs ceil(tokens / max_tokens) passes, not one per chunk."""
            run: list[int] = []
            run_start = 0

            def flush(sample_with=None):
                nonlocal gate, run
                out = None
                if run:
                    out = self._prefill_tokens(run, run_start, req.block_table, sample_with, gate=gate)
                    gate = None
                    run = []
                return out

            ctx = 0
            for c, off, ok in zip(req.chunks, offsets, found):
                blocks_of_chunk = set(req.block_table[off // bt : (off + len(c)) // bt])
                if not ok or (blocks_of_chunk & failed_blocks):
                    if run and run_start + len(run) != off:
                        flush()
                    if not run:
                        run_start = off
                    run.extend(c)
                    if req.store_misses and not ok:
                        if off == 0:
                            if (c, off) not in in_place:
                                in_place.append((c, off))  # saw no context: this IS the chunk's own KV
                        elif c not in standalone:
                            standalone.append(c)
                    if ok and failed_blocks:  # counted as restored by the first pass
                        req.restored_chunks -= 1
                        req.restored_bytes -= (len(c) // bt) * self.geo.slot_size
                else:
                    flush()
                    if not failed_blocks:
                        req.restored_chunks += 1
                        req.restored_bytes += (len(c) // bt) * self.geo.slot_size
                        if self.repair_tokens > 0 and off > 0:
                            self._prefill_tokens(c[: min(self.repair_tokens, len(c))], off, req.block_table, gate=gate)
                            gate = None
                ctx = off + len(c)
            if run and run_start + len(run) != ctx:
                flush()
            if not run:
                run_start = ctx
            run.extend(req.query)
            return flush(sample)

        # A missed chunk behind other context was just computed attending to that context; the
        # store keeps chunks under a key of their own tokens only, so what is stored must be the
        # chunk computed alone (as `store_chunk` does).  Those are recomputed after the first
        # token has gone out, between steps.
        standalone: list[Sequence[int]] = []
        # A missed chunk at offset 0 is stored from the request's own blocks, once the first token is out.
        in_place: list[tuple[Sequence[int], int]] = []
        # 3. compute what was not restored, then the query
        first = compute(set(), gate)
        if self._restore_stream is not None:
            self._ev[2].record(self._restore_stream)
        # a load that failed on any rank (rare): recompute those chunks and the query once more
        failed_blocks = self.worker.take_load_errors()
        if self.tp_ctx is not None and meta.reqs_to_load:
            failed_blocks = set().union(*self.tp_ctx.gather_object(sorted(failed_blocks)))
        elif self.pp_link is not None and meta.reqs_to_load:
            failed_blocks = set().union(*self.pp_link.gather_object(sorted(failed_blocks)))
        if failed_blocks:
            first = compute(set(failed_blocks), None)
        self._ev[3].record()
        token = self._tokens_out(first, 1)[0]  # device -> host read of the step's result
        t_end = time.perf_counter()
        self.worker.check_load_status()
        req.generated.append(token)
        req.context_len = total
        req.ttft_ms = (t_end - t_start) * 1e3
        req.first_token_time = t_end
        req.ttft_device_ms = self._ev[0].elapsed_time(self._ev[3])
        req.timings = {
            "plan_ms": (t_plan - t_start) * 1e3,
            "restore_ms": (t_restore - t_plan) * 1e3,  # host time to issue the loads (the pieces overlap the forward)
            "restore_device_ms": (self._ev[1].elapsed_time(self._ev[2])
                                  if ticket is not None and self._restore_stream is not None else 0.0),
            "compute_ms": (t_end - t_restore) * 1e3,
            "io_wait_ms": ticket.io_wait_ms if ticket is not None else 0.0,
            "io_bytes": ticket.io_bytes if ticket is not None else 0,
            "h2d_bytes": self.h2d_bytes + self.kv_backend.h2d_bytes - h2d0,
        }
        metrics.observe("engine.ttft_ms", req.ttft_ms)
        for c, off in in_place:
            self._store_in_place(req, c, off)
        if self.sched is not None:
            self.sched.request_finished(req.req_id)
        for c in standalone:
            if len(c) // bt <= self.blocks.num_free:
                self.store_chunk(c)
        if req.finished():
            self._finish(req)
        else:
            self.running.append(req)

    def _store_in_place(self, req: RagRequest, chunk: Sequence[int], off: int) -> None:
        """Save a chunk that was just computed inside the request.  Only valid for ``off == 0``:
        further back the KV has attended to the request's earlier chunks and is not the chunk's own."""
        bt = self.cfg.block_tokens
        blocks = req.block_table[off // bt : (off + len(chunk)) // bt]
        meta = ConnectorMeta()
        sub = f"{req.req_id}.s{off}"
        if self.sched is not None:
            if self.sched.reserve_chunk_store(sub, chunk, blocks, pos_offset=off) is not None:
                meta = self.sched.build_connector_meta([sub])
        meta = self._bcast(meta)
        self._save(meta)
        if self.sched is not None:
            self.sched.request_finished(sub)

    @staticmethod
    def decode_bucket(n: int, cap: int) -> int:
        """Batch sizes are rounded up to powers of two so that a handful of captured graphs serve
        every decode step (a batch that grows and shrinks by one would otherwise meet a new shape,
        run eagerly and capture, at almost every step)."""
        b = 1
        while b < n:
            b *= 2
        return min(b, cap) if cap >= n else n

    def _decode_step(self) -> None:
        batch = self.running[: self.runner.max_seqs]
        seqs = [{"tokens": [r.generated[-1]], "start_pos": r.context_len + len(r.generated) - 1,
                 "block_table": r.block_table, "temperature": r.temperature, "seed": r.step_seed(),
                 "top_k": r.top_k, "top_p": r.top_p} for r in batch]
        # padding rows repeat the first sequence: they rewrite the same KV entry with the same
        # value and their samples are dropped
        seqs += [seqs[0]] * (self.decode_bucket(len(seqs), self.runner.max_seqs) - len(seqs))
        inp = self.runner.stage_inputs(seqs)
        self.h2d_bytes += self.runner.h2d_bytes
        out = self._tokens_out(self.runner.forward(inp), len(batch))
        for r, tok in zip(batch, out):
            r.generated.append(int(tok))
            if r.finished():
                self._finish(r)

    def _finish(self, req: RagRequest) -> None:
        req.done = True
        if req in self.running:
            self.running.remove(req)
        self.blocks.free(req.block_table)
        room = sum(len(c) for c in req.asked) // self.cfg.block_tokens <= self.blocks.num_free
        if self.compose_after > 0 and req.asked and room:  # (no room for the prefill now: next sighting)
            # a chunk combination seen often enough is computed from scratch (its chunks attending to
            # one another) and stored whole, here between two steps
            combo = self._bcast(self.sched.note_composition(req.asked, self.compose_after)
                                if self.sched is not None else None)
            if combo is not None:
                self.store_chunk(combo)

    def generate(self, chunks: Sequence[Sequence[int]], query: Sequence[int], max_new_tokens: int = 1,
                 store_misses: bool = False, on_token=None, temperature: float = 0.0, seed: int = 0,
                 stop_token_ids: Sequence[int] = (), top_k: int = 0, top_p: float = 1.0) -> RagRequest:
        """Serve one request to completion (the call a user of the engine makes).

        ``on_token(token_id)`` is called after each engine step with every token the step added
        (a streaming front end sends the first one on as soon as the prefill step has ended)."""
        req = self.submit(RagRequest([list(c) for c in chunks], list(query), max_new_tokens, store_misses=store_misses,
                                     temperature=float(temperature), seed=int(seed), top_k=int(top_k),
                                     top_p=float(top_p), stop_token_ids=tuple(int(t) for t in stop_token_ids)))
        sent = 0
        while not req.done:
            self.step()
            if on_token is not None:
                for tok in req.generated[sent:]:
                    on_token(int(tok))
                sent = len(req.generated)
        if req.error is not None:
            raise MemoryError(req.error)
        return req

    def close(self) -> None:
        if self.worker is not None:
            self.worker.shutdown()
        if self.sched is not None:
            self.sched.close()
        if self.tp_ctx is not None:
            self.tp_ctx.close()
