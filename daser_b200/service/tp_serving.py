"""Serving a tensor-parallel engine behind one HTTP front end.

The engine's calls are collective: every rank has to run ``store_chunk`` / ``generate`` with the
same arguments, in the same order.  Only rank 0 sees HTTP requests, so it leads: each call is
first announced to the other ranks over the group's CPU (gloo) channel, then executed locally;
the other ranks sit in :func:`follower_loop` and replay what they are told.

::

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m daser_b200.service --engine native --native-device cuda --native-model llama3-70b ...

The reference's service talks to a remote stock vLLM and leaves tensor parallelism to it
(``daser/service/vllm_client.py:15-146``); its own connector is not rank aware at all.

An engine loop (``engine/loop.py``) on the leader drives ``submit`` / ``step`` instead of
``generate``; both are announced the same way, so the followers' queues mirror the leader's and a
step batches the same requests on every rank.

Failure handling: a follower that cannot be reached makes the announcement itself fail (the
gloo broadcast times out or raises); the leader then marks the engine unavailable, which the
front end reports through ``/health`` (see ``NativeEngineClient``).  ``shutdown`` tells the
followers to leave between steps.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

from daser_b200.logging import init_logger

logger = init_logger(__name__)

Broadcast = Callable[[Any], Any]  # leader: sends and returns its argument; follower: returns what was sent

CMD_STORE = "store_chunk"
CMD_GENERATE = "generate"
CMD_WARM_UP = "warm_up"
CMD_SUBMIT = "submit"
CMD_STEP = "step"
CMD_ABORT = "abort"
CMD_STOP = "stop"


class TPLeaderEngine:
    """Rank 0's view of the engine: announces every collective call, then runs it."""

    def __init__(self, engine: Any, broadcast: Broadcast) -> None:
        self._engine = engine
        self._bcast = broadcast
        self._stopped = False

    @property
    def cfg(self):
        return self._engine.cfg

    @property
    def device(self):
        return getattr(self._engine, "device", None)

    def _announce(self, *cmd: Any) -> None:
        if self._stopped:
            raise RuntimeError("the tensor-parallel engine was shut down")
        self._bcast(tuple(cmd))

    def store_chunk(self, tokens: Sequence[int]) -> str:
        tokens = list(tokens)
        self._announce(CMD_STORE, tokens)
        return self._engine.store_chunk(tokens)

    def generate(self, chunks: Sequence[Sequence[int]], query: Sequence[int], max_new_tokens: int = 1,
                 on_token: Optional[Callable[[int], None]] = None, **kw: Any):
        chunks = [list(c) for c in chunks]
        query = list(query)
        self._announce(CMD_GENERATE, chunks, query, int(max_new_tokens), dict(kw))
        if on_token is not None:  # a local observer: the followers neither need nor could receive it
            kw = dict(kw, on_token=on_token)
        return self._engine.generate(chunks, query, max_new_tokens=max_new_tokens, **kw)

    # iteration-level calls (an engine loop drives these instead of `generate`)
    def submit(self, req: Any) -> Any:
        self._announce(CMD_SUBMIT, [list(c) for c in req.chunks], list(req.query), int(req.max_new_tokens),
                       bool(req.store_misses), float(req.temperature), int(req.seed), tuple(req.stop_token_ids),
                       int(req.top_k), float(req.top_p))
        return self._engine.submit(req)

    def has_work(self) -> bool:
        return self._engine.has_work()  # the same on every rank: they hold the same queues

    def step(self) -> None:
        self._announce(CMD_STEP)
        self._engine.step()

    def abort(self, req_id: str) -> bool:
        self._announce(CMD_ABORT, req_id)  # request ids are assigned in submit order: the same on every rank
        return self._engine.abort(req_id)

    def warm_up(self, *args: Any, **kw: Any) -> None:
        self._announce(CMD_WARM_UP, list(args), dict(kw))
        self._engine.warm_up(*args, **kw)

    def close(self) -> None:
        """Tell the followers to leave (between steps), then close the local engine."""
        if not self._stopped:
            try:
                self._bcast((CMD_STOP,))
            except Exception as exc:  # followers already gone
                logger.warning("[SERVICE] could not announce shutdown to the followers: %r", exc)
            self._stopped = True
        self._engine.close()


def follower_loop(engine: Any, broadcast: Broadcast, on_step: Optional[Callable[[tuple], None]] = None) -> int:
    """Replay the leader's calls until it says stop; returns the number of calls executed."""
    steps = 0
    while True:
        cmd = broadcast(None)
        if not isinstance(cmd, tuple) or not cmd:
            raise RuntimeError(f"malformed command from the leader: {cmd!r}")
        if on_step is not None:
            on_step(cmd)
        op = cmd[0]
        if op == CMD_STOP:
            engine.close()
            return steps
        if op == CMD_STORE:
            engine.store_chunk(cmd[1])
        elif op == CMD_GENERATE:
            _, chunks, query, max_new, kw = cmd
            engine.generate(chunks, query, max_new_tokens=max_new, **kw)
        elif op == CMD_SUBMIT:
            from daser_b200.engine.request import RagRequest

            _, chunks, query, max_new, store_misses, temperature, seed, stops, top_k, top_p = cmd
            engine.submit(RagRequest(chunks, query, max_new, store_misses=store_misses, temperature=temperature,
                                     seed=seed, stop_token_ids=tuple(stops), top_k=top_k, top_p=top_p))
        elif op == CMD_STEP:
            engine.step()
        elif op == CMD_ABORT:
            engine.abort(cmd[1])
        elif op == CMD_WARM_UP:
            engine.warm_up(*cmd[1], **cmd[2])
        else:
            raise RuntimeError(f"unknown command from the leader: {op!r}")
        steps += 1
