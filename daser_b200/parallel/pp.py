"""Pipeline parallelism: contiguous layer ranges on successive processes, activations handed on
with point-to-point sends.

The reference has no pipeline parallelism, and the stack it is benchmarked with never enables
vLLM's.  What a chunk-KV service has to add to the textbook scheme is the cache side: a stored
chunk holds the KV of EVERY layer, but a stage only has, and only needs, its own layers.  Here
each stage keeps a store file of its own with slots sized for the widest stage
(``<store>.pp<stage>of<stages>``), saves and restores only its layers there, and a chunk
becomes visible when all stages have committed their part (the control plane's multi-part
commit, ``server/ipc_server.py::_handle_commit_chunk``).  The control plane therefore runs with
the slot size :func:`stage_geometry` gives, and one ring slot still means one token block.

Scheduling lives on stage 0 (the only process that plans, reserves and finishes requests);
the other stages receive the step's connector metadata with the step.  Activations travel as
``[T, hidden]`` tensors over ``torch.distributed`` point-to-point calls (gloo between CPU
processes, NCCL p2p between GPUs), sent asynchronously: a stage posts its send and starts on the
next piece of the request (a missing chunk, then the query) while the next stage works on the
previous one.  The sampled token goes back from the last stage to all.

:class:`PipelineCpuEngine` runs the oracle model (``models/llama.py::reference_forward`` on a
layer range) and is what the CPU tests drive; it keeps the public calls of
:class:`~daser_b200.engine.rag_cpu.CpuRagEngine`.  On GPUs the same scheme is a mode of the native
engine: ``GpuRagEngine(..., pp_link=StageLink(group))`` runs this stage's layers on the sm_100a
kernels (``GpuModelRunner(layer_range=...)``), receives the residual stream with an NCCL receive
in front of its first layer group, posts it on behind its last, and the last stage broadcasts
the sampled tokens (``tests/pp_worker.py``).
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch
import torch.distributed as dist

from daser_b200.connector.core import SchedulerHalf, TorchKVBackend, WorkerHalf
from daser_b200.engine.rag_cpu import BlockAllocator, CpuRagEngine
from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import LlamaConfig, LlamaWeights, TorchPagedKV, reference_forward


def partition_layers(num_layers: int, stages: int) -> list[range]:
    """Contiguous, balanced layer ranges; earlier stages take the remainder (the last stage also
    carries the final norm and the output projection)."""
    if stages < 1 or stages > num_layers:
        raise ValueError(f"cannot split {num_layers} layers into {stages} stages")
    base, extra = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def stage_geometry(cfg: LlamaConfig, stages: int, dtype_bytes: int = 4, codec_name: str = "raw") -> KVGeometry:
    """Slot geometry of every stage's store file: the layer count of the widest stage."""
    widest = max(len(r) for r in partition_layers(cfg.num_layers, stages))
    return KVGeometry(widest, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, dtype_bytes, codec_name)


def stage_store_path(store_path: str, stage: int, stages: int) -> str:
    return f"{store_path}.pp{stage}of{stages}"


class StageLink:
    """Point-to-point plumbing between the stages of one pipeline (one process per stage)."""

    def __init__(self, group: Any = None) -> None:
        self.group = group if group is not None else dist.group.WORLD
        self.stage = dist.get_rank(self.group)
        self.stages = dist.get_world_size(self.group)
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        self._inflight: list[tuple[Any, torch.Tensor]] = []

    def _global(self, stage: int) -> int:
        return dist.get_global_rank(self.group, stage)

    def send_next(self, t: torch.Tensor) -> None:
        """Post the hand-over and return: the tensor stays referenced until :meth:`drain`."""
        t = t.contiguous()
        self._inflight.append((dist.isend(t, self._global(self.stage + 1), group=self.group), t))

    def recv_prev(self, shape: Sequence[int], dtype: torch.dtype, device: Any = "cpu") -> torch.Tensor:
        buf = torch.empty(tuple(shape), dtype=dtype, device=device)
        dist.recv(buf, self._global(self.stage - 1), group=self.group)
        return buf

    def recv_prev_into(self, buf: torch.Tensor) -> torch.Tensor:
        """Receive the previous stage's hand-over into an existing (persistent) buffer."""
        dist.recv(buf, self._global(self.stage - 1), group=self.group)
        return buf

    def drain(self) -> None:
        for work, _ in self._inflight:
            work.wait()
        self._inflight.clear()

    def from_stage(self, obj: Any, stage: int) -> Any:
        """``obj`` of ``stage`` on every stage (pickled; for plans and small results)."""
        box = [obj]
        dist.broadcast_object_list(box, src=self._global(stage), group=self.group)
        return box[0]

    def barrier(self) -> None:
        if dist.get_backend(self.group) == "nccl":
            dist.barrier(group=self.group, device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier(group=self.group)

    def gather_object(self, obj: Any) -> list:
        """Every stage's ``obj`` in stage order, on every stage."""
        out: list = [None] * self.stages
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def tokens_from_last(self, tokens: Optional[torch.Tensor], n: int, device: Any = "cpu") -> list[int]:
        """The last stage's ``n`` sampled tokens as a list on every stage (one broadcast, one read)."""
        buf = torch.empty(n, dtype=torch.int64, device=device)
        if self.last:
            buf.copy_(tokens[:n])
        dist.broadcast(buf, self._global(self.stages - 1), group=self.group)
        self.drain()  # the tokens exist, so every hand-over that led to them has completed
        return [int(t) for t in buf.tolist()]

    def token_from_last(self, token: Optional[int], device: Any = "cpu") -> int:
        t = torch.tensor([token if token is not None else -1], dtype=torch.int64, device=device)
        dist.broadcast(t, self._global(self.stages - 1), group=self.group)
        return int(t.item())


class PipelineCpuEngine(CpuRagEngine):
    """One pipeline stage of the oracle engine; every stage makes the same public calls with the
    same arguments (stage 0 plans, the last stage samples).  Results that exist only on the last
    stage (``RequestResult.logits``) are ``None`` elsewhere."""

    def __init__(self, cfg: LlamaConfig, socket_path: str, store_path: str, group: Any = None,
                 num_blocks: int = 512, codec_name: str = "raw", dtype: torch.dtype = torch.float32, seed: int = 0,
                 io_backend: str = "auto", model_id: str = "default", compose_after: int = 0,
                 repair_tokens: int = 0) -> None:
        self.cfg = cfg
        self.compose_after = compose_after
        self.repair_tokens = repair_tokens
        self.link = StageLink(group)
        st, n = self.link.stage, self.link.stages
        self.layers = partition_layers(cfg.num_layers, n)[st]
        # Every stage draws the same random model and drops what it does not run (a loader of
        # real weights would read only its slice); the embedding stays as the device anchor.
        self.weights = LlamaWeights.random(cfg, "cpu", dtype, seed=seed)
        self.weights.layers = [lw if i in self.layers else None for i, lw in enumerate(self.weights.layers)]
        if not self.link.last:
            self.weights.lm_head = None
        self.geo = stage_geometry(cfg, n, {torch.float32: 4, torch.bfloat16: 2}[dtype], codec_name)
        self.pool = TorchPagedKV(cfg, num_blocks, dtype, num_layers=self.geo.num_layers)
        self.blocks = BlockAllocator(num_blocks)  # every stage allocates in step: identical tables
        self.sched = SchedulerHalf(socket_path, cfg.block_tokens, model_id) if self.link.first else None
        self.host = None
        self.worker = WorkerHalf(socket_path, stage_store_path(store_path, st, n), self.geo,
                                 TorchKVBackend(self.geo, self.pool.data, cfg.inv_freq()), io_backend=io_backend)
        if n > 1:
            self.worker.commit_parts = (st, n)
        self._req = 0
        self.waiting, self.running = [], []

    # -- the hooks of CpuRagEngine --------------------------------------------------------------------
    def _lead(self, fn):
        out: Any = None
        if self.link.first:
            try:
                out = ("ok", fn())
            except Exception as exc:  # the other stages must not wait for a plan that never comes
                out = ("error", f"{type(exc).__name__}: {exc}")
        kind, value = self.link.from_stage(out, 0)
        if kind == "error":
            raise RuntimeError(f"stage 0 failed: {value}")
        return value

    def _forward(self, tokens: Sequence[int], positions: torch.Tensor, table: torch.Tensor, context_len: int,
                 return_logits: bool = True) -> Optional[torch.Tensor]:
        tokens = list(tokens)
        hidden = None
        if not self.link.first:
            hidden = self.link.recv_prev((len(tokens), self.cfg.hidden), torch.float32)
        out = reference_forward(self.weights, torch.tensor(tokens), positions, self.pool, table, context_len,
                                return_logits=return_logits, layers=self.layers, hidden_in=hidden)
        if self.link.last:
            return out
        self.link.send_next(out)  # asynchronous: this stage moves on to the next piece
        return None

    def _sample(self, logits: Optional[torch.Tensor], req=None) -> int:
        token = self.link.token_from_last(super()._sample(logits, req) if self.link.last else None)
        self.link.drain()  # the token exists, so every hand-over that led to it has completed
        return token

    def _step(self, meta, fn):
        try:
            return super()._step(meta, fn)
        finally:
            self.link.drain()

    def close(self) -> None:
        self.link.drain()
        self.worker.shutdown()
        if self.sched is not None:
            self.sched.close()
