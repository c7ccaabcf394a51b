"""One thread that owns the engine and keeps it stepping, so that concurrent callers share steps.

``engine.generate`` serves one request from its prefill to its last token; callers that arrive
meanwhile wait for the whole of it.  The engines schedule per iteration, though
(``submit`` / ``step``: the prefill of the oldest waiting request first, else one decode step for
every running request together), so a front end that hands requests over as they arrive gets
continuous batching: a new request's prefill slips in between two decode steps of the others, and
the decode steps carry every running request at once.

:class:`EngineLoop` is that hand-over.  Any thread may call :meth:`submit` (returns a
``concurrent.futures.Future`` of the finished request; ``on_token`` is called from the loop thread
as tokens are sampled) or :meth:`call` (runs an engine method such as ``store_chunk`` between two
steps).  The engine itself is only ever touched by the loop thread, which matters for the GPU
engine: CUDA graphs, its streams and the tensor-parallel announcements all assume one caller.

The reference has no engine of its own (it forwards to a remote vLLM, which has such a loop
inside: ``daser/service/vllm_client.py:62-126``).
"""

from __future__ import annotations

import queue
import threading
from concurrent.futures import Future
from typing import Any, Callable, Optional, Sequence

from daser_b200 import metrics
from daser_b200.engine.request import RagRequest
from daser_b200.logging import init_logger

logger = init_logger(__name__)


class _Tracked:
    __slots__ = ("req", "future", "on_token", "sent")

    def __init__(self, req: RagRequest, future: Future, on_token: Optional[Callable[[int], None]]) -> None:
        self.req, self.future, self.on_token, self.sent = req, future, on_token, 0


def _settle(fut: Future, result: Any = None, exc: Optional[BaseException] = None) -> None:
    """Complete ``fut`` unless its owner got there first (an asyncio wrapper that was cancelled
    cancels the future underneath it at once, before the loop thread hears of it)."""
    try:
        if fut.done():
            return
        if exc is not None:
            fut.set_exception(exc)
        else:
            fut.set_result(result)
    except Exception:  # InvalidStateError: cancelled between the check and the call
        pass


class QueueFull(RuntimeError):
    """More requests in flight than the loop was told to take: the caller should come back later."""


class EngineLoop:
    def __init__(self, engine: Any, idle_wait_s: float = 0.05, max_in_flight: int = 0) -> None:
        if not (hasattr(engine, "submit") and hasattr(engine, "step") and hasattr(engine, "has_work")):
            raise TypeError("the engine has no submit / step / has_work: it cannot be stepped by a loop")
        self.engine = engine
        self._idle_wait = idle_wait_s
        self._inbox: queue.Queue = queue.Queue()
        self._tracked: list[_Tracked] = []
        # back-pressure: requests submitted and not yet finished (queued, waiting, running); above
        # `max_in_flight` (0 = no limit) a submit fails at once instead of queueing without bound
        self._max_in_flight = max_in_flight
        self._in_flight = 0
        self._count_lock = threading.Lock()
        self._stop = False
        self.failed: Optional[BaseException] = None
        self.steps = 0
        self.max_batch = 0  # most requests in flight at once (prefilled, still decoding)
        self._thread = threading.Thread(target=self._run, name="daser-engine", daemon=True)
        self._thread.start()

    # -- any thread ----------------------------------------------------------------------------------
    def submit(self, chunks: Sequence[Sequence[int]], query: Sequence[int], max_new_tokens: int = 1,
               on_token: Optional[Callable[[int], None]] = None, **fields: Any) -> Future:
        fut: Future = Future()
        if self._stop or self.failed is not None:
            fut.set_exception(RuntimeError(f"engine loop is not running: {self.failed or 'closed'}"))
            return fut
        # what the engine would only find out inside a step (where a failure takes the others down)
        bt = getattr(getattr(self.engine, "cfg", None), "block_tokens", None)
        if bt and any(len(c) % bt for c in chunks):
            fut.set_exception(ValueError(f"cached segments must be whole blocks of {bt} tokens"))
            return fut
        if len(query) < 1 or int(max_new_tokens) < 1:
            fut.set_exception(ValueError("a request needs at least one query token and one token to generate"))
            return fut
        with self._count_lock:
            if self._max_in_flight and self._in_flight >= self._max_in_flight:
                fut.set_exception(QueueFull(f"{self._in_flight} requests in flight (limit {self._max_in_flight})"))
                return fut
            self._in_flight += 1
        fut.add_done_callback(self._one_less)
        req = RagRequest([list(c) for c in chunks], list(query), int(max_new_tokens), **fields)
        self._inbox.put(("submit", _Tracked(req, fut, on_token)))
        return fut

    def _one_less(self, _fut: Future) -> None:
        with self._count_lock:
            self._in_flight -= 1

    def cancel(self, fut: Future) -> None:
        """Stop working on the request behind ``fut`` (as returned by :meth:`submit`): it leaves the
        engine between two steps and the future fails with ``CancelledError``-like ``RuntimeError``.
        Harmless when the request has finished."""
        if not fut.done():
            self._inbox.put(("cancel", fut))

    def call(self, method: str, *args: Any, **kw: Any) -> Future:
        """Run ``engine.<method>(*args, **kw)`` on the loop thread, between two steps."""
        fut: Future = Future()
        if self._stop or self.failed is not None:
            fut.set_exception(RuntimeError(f"engine loop is not running: {self.failed or 'closed'}"))
            return fut
        self._inbox.put(("call", (fut, method, args, kw)))
        return fut

    def close(self, timeout_s: float = 60.0) -> None:
        """Finish what is in flight, then stop the thread (the engine is left open).  What is still
        running after ``timeout_s`` is aborted, so that the caller may close the engine after this."""
        self._stop = True
        self._inbox.put(("wake", None))
        self._thread.join(timeout_s)
        if self._thread.is_alive():
            self._inbox.put(("abort_all", None))
            self._thread.join(timeout_s)

    # -- the loop thread ---------------------------------------------------------------------------
    def _take(self, block: bool) -> bool:
        try:
            kind, item = self._inbox.get(timeout=self._idle_wait) if block else self._inbox.get_nowait()
        except queue.Empty:
            return False
        if kind == "submit":
            self.engine.submit(item.req)
            self._tracked.append(item)
        elif kind == "abort_all":
            for t in list(self._tracked):
                if hasattr(self.engine, "abort"):
                    self.engine.abort(t.req.req_id)
                _settle(t.future, exc=RuntimeError("engine loop closed"))
            if hasattr(self.engine, "abort"):
                self._tracked.clear()
        elif kind == "cancel":
            for t in self._tracked:
                if t.future is item:
                    if hasattr(self.engine, "abort"):
                        self.engine.abort(t.req.req_id)
                    else:
                        t.on_token = None  # an engine without abort runs the request out, unobserved
                        break
                    self._tracked.remove(t)
                    _settle(t.future, exc=RuntimeError("request cancelled"))
                    break
        elif kind == "call":
            fut, method, args, kw = item
            try:
                _settle(fut, result=getattr(self.engine, method)(*args, **kw))
            except Exception as exc:  # the caller's error, not the loop's
                _settle(fut, exc=exc)
        return True

    def _report(self) -> None:
        for t in list(self._tracked):
            if t.on_token is not None:
                for tok in t.req.generated[t.sent:]:
                    try:
                        t.on_token(int(tok))
                    except Exception as exc:  # a closed client must not stop the others
                        logger.warning("[ENGINE] token callback failed: %r", exc)
                        t.on_token = None
                        break
            t.sent = len(t.req.generated)
            if t.req.done:
                self._tracked.remove(t)
                if t.req.error is not None:  # given up alone (it can never fit): the others go on
                    _settle(t.future, exc=MemoryError(t.req.error))
                else:
                    _settle(t.future, result=t.req)

    def _fail(self, exc: BaseException) -> None:
        self.failed = exc
        for t in self._tracked:
            _settle(t.future, exc=exc)
        self._tracked.clear()
        while True:  # whoever queued meanwhile
            try:
                kind, item = self._inbox.get_nowait()
            except queue.Empty:
                break
            fut = item.future if kind == "submit" else (item[0] if kind == "call" else None)  # cancels: nothing to tell
            if fut is not None:
                _settle(fut, exc=exc)

    def _run(self) -> None:
        try:
            dev = getattr(self.engine, "device", None)
            if dev is not None and getattr(dev, "type", "") == "cuda":
                import torch

                torch.cuda.set_device(dev)  # the current device is per thread; the engine was built elsewhere
            while True:
                while self._take(block=False):  # everything that arrived since the last step
                    pass
                if self.engine.has_work():
                    self.engine.step()
                    self.steps += 1
                    self.max_batch = max(self.max_batch, len(self._tracked))
                    metrics.set_gauge("engine.loop_in_flight", len(self._tracked))
                    self._report()
                elif self._stop:
                    return
                else:
                    self._take(block=True)
        except BaseException as exc:  # a failed step invalidates every request in flight
            logger.error("[ENGINE] loop stopped: %r", exc)
            self._fail(exc)
