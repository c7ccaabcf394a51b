"""Queue handling shared by the CUDA engine and the oracle engine: admission against the KV pool,
and dropping a request between two steps.  (One implementation, so that the CPU tests of the oracle
engine also cover what the CUDA engine does.)

The reference has no scheduler of its own: requests are queued, admitted and preempted inside the
remote vLLM (``vllm/v1/core/sched/scheduler.py``), which its service reaches over HTTP
(``daser/service/vllm_client.py:62-126``)."""

from __future__ import annotations

from typing import Optional

from daser_b200 import metrics

START, WAIT, REJECT = "start", "wait", "reject"


class SchedulingMixin:
    """Expects ``waiting`` / ``running`` (lists of :class:`~daser_b200.engine.request.RagRequest`),
    ``blocks`` (a block allocator) and ``cfg.block_tokens`` on the engine."""

    max_blocks_per_seq: Optional[int] = None  # a limit of the model runner's block tables, if any

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _admission(self) -> str:
        """What to do with the oldest waiting request.  ``start``: its blocks (context plus the whole
        generation, reserved up front so that a running request is never starved) are free.
        ``wait``: they are not, but running requests will free theirs: decode instead.  ``reject``:
        it cannot fit even an idle engine, or exceeds the runner's blocks per sequence; it has been
        taken off the queue and marked (``error``, ``done``), the others go on.  The decision depends
        on queue and pool state only, which every tensor-parallel rank shares."""
        req = self.waiting[0]
        need = req.blocks_needed(self.cfg.block_tokens)
        why = None
        if self.max_blocks_per_seq is not None and need > self.max_blocks_per_seq:
            why = f"{need} KV blocks exceed the limit of {self.max_blocks_per_seq} per sequence"
        elif need > self.blocks.num_free and not self.running:
            why = f"{need} KV blocks needed, the pool has {self.blocks.num_free} free of {self.blocks.num_blocks}"
        if why is not None:
            self.waiting.pop(0)
            req.error, req.done = why, True
            metrics.inc("engine.requests_rejected")
            return REJECT
        return START if need <= self.blocks.num_free else WAIT

    def abort(self, req_id: str) -> bool:
        """Drop a waiting or running request between two steps (a client that went away); its blocks
        go back to the pool.  False when the request is unknown or already finished."""
        for queue in (self.waiting, self.running):
            for req in queue:
                if req.req_id == req_id:
                    queue.remove(req)
                    if req.block_table:
                        self.blocks.free(req.block_table)
                    req.error, req.done = "aborted", True
                    metrics.inc("engine.requests_aborted")
                    return True
        return False
