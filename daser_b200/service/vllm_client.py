"""Engine clients used by the service.

Capability parity: ``daser/service/vllm_client.py:15-146`` — :class:`VLLMClient` posts
token-id prompts to an OpenAI-compatible ``/v1/completions`` (``prefill`` = one token at
temperature 0, ``completion`` with defaults ``max_tokens=256, temperature=0.7`` overridden
by the caller, ``health`` never raises, 300 s timeout).

Added: :class:`NativeEngineClient` serves the same three calls from the in-process engine
(:mod:`daser_b200.engine`), and additionally accepts *segments* so cached document chunks
are restored at their offsets instead of being recomputed.
"""

from __future__ import annotations

import asyncio
import random
from typing import Any, Optional, Sequence


class VLLMClient:
    def __init__(self, base_url: str, model: str, timeout_s: float = 300.0) -> None:
        import httpx

        self._base = base_url.rstrip("/")
        self._model = model
        self._http = httpx.AsyncClient(timeout=timeout_s)

    async def __aenter__(self) -> "VLLMClient":
        return self

    async def __aexit__(self, *exc: Any) -> None:
        await self.close()

    @property
    def model(self) -> str:
        return self._model

    async def close(self) -> None:
        await self._http.aclose()

    async def _post_completions(self, payload: dict[str, Any]) -> dict[str, Any]:
        resp = await self._http.post(f"{self._base}/v1/completions", json=payload)
        resp.raise_for_status()
        return resp.json()

    async def prefill(self, tokens: list[int]) -> None:
        """Run the prompt through the engine so the connector stores its KV."""
        await self._post_completions({"model": self._model, "prompt": tokens, "max_tokens": 1, "temperature": 0.0})

    async def completion(self, tokens: list[int], gen_params: Optional[dict[str, Any]] = None,
                         segments: Optional[Sequence[Sequence[int]]] = None) -> dict[str, Any]:
        payload: dict[str, Any] = {"model": self._model, "prompt": tokens, "max_tokens": 256, "temperature": 0.7}
        payload.update(gen_params or {})
        return await self._post_completions(payload)

    async def completion_stream(self, tokens: list[int], gen_params: Optional[dict[str, Any]] = None,
                                segments: Optional[Sequence[Sequence[int]]] = None):
        """The same request with ``"stream": true``: yields ``{"token_ids", "text"}`` per
        server-sent event and a last ``{"done": True, "usage": ...}`` (the shape of
        :meth:`NativeEngineClient.completion_stream`)."""
        import json

        payload: dict[str, Any] = {"model": self._model, "prompt": tokens, "max_tokens": 256, "temperature": 0.7}
        payload.update(gen_params or {})
        payload["stream"] = True
        usage: dict[str, Any] = {}
        async with self._http.stream("POST", f"{self._base}/v1/completions", json=payload) as resp:
            resp.raise_for_status()
            async for line in resp.aiter_lines():
                if not line.startswith("data: "):
                    continue
                data = line[6:].strip()
                if data == "[DONE]":
                    break
                obj = json.loads(data)
                if "error" in obj:
                    raise RuntimeError(str(obj["error"].get("message", obj["error"])))
                usage = obj.get("usage") or usage
                choice = (obj.get("choices") or [{}])[0]
                if choice.get("text") or choice.get("token_ids"):
                    yield {"token_ids": list(choice.get("token_ids") or []), "text": choice.get("text", "")}
        yield {"done": True, "usage": usage}

    async def health(self) -> bool:
        try:
            resp = await self._http.get(f"{self._base}/health")
            return resp.status_code == 200
        except Exception:
            return False


class _NoLock:
    async def __aenter__(self) -> None:
        return None

    async def __aexit__(self, *exc: Any) -> None:
        return None


class NativeEngineClient:
    """The in-process engine behind the same interface.

    ``engine`` is a :class:`~daser_b200.engine.rag_cpu.CpuRagEngine` or
    :class:`~daser_b200.engine.rag_gpu.GpuRagEngine`; ``detokenize`` turns generated ids
    into text.  Engine calls run in a worker thread so the event loop (which also serves
    the control plane) stays responsive.
    """

    def __init__(self, engine: Any, detokenize, model: str = "native", pad_token: int = 0,
                 batching: bool = False, eos_token_ids: Sequence[int] = (), max_in_flight: int = 0) -> None:
        self._engine = engine
        self.eos_token_ids = tuple(int(t) for t in eos_token_ids)  # generation stops at these
        self._detok = detokenize
        self._model = model
        self._pad = pad_token
        self._lock = asyncio.Lock()
        self._failed: Optional[str] = None  # set once the engine lost a tensor-parallel peer
        # batching: one thread keeps the engine stepping and concurrent requests share its steps
        # (continuous batching); without it requests are served one after the other
        self._loop = None
        if batching:
            from daser_b200.engine.loop import EngineLoop

            self._loop = EngineLoop(engine, max_in_flight=max_in_flight)

    @property
    def model(self) -> str:
        return self._model

    async def close(self) -> None:
        if self._loop is not None:
            await asyncio.get_running_loop().run_in_executor(None, self._loop.close)

    async def health(self) -> bool:
        """False once a step failed with a lost peer or an invalid device status: the group has
        to be restarted, `/health` degrades and `/infer` answers 502 until then."""
        if self._loop is not None and self._loop.failed is not None:
            return False
        return self._failed is None

    def _guard(self, fn, *args):
        if self._failed is not None:
            raise RuntimeError(f"engine unavailable: {self._failed}")
        dev = getattr(self._engine, "device", None)
        if dev is not None and getattr(dev, "type", "") == "cuda":
            import torch

            torch.cuda.set_device(dev)  # worker threads start on device 0: use the engine's
        try:
            return fn(*args)
        except Exception as exc:
            if type(exc).__name__ == "PeerLost":
                self._failed = str(exc)
            raise

    async def prefill(self, tokens: list[int]) -> None:
        if self._loop is not None:
            await asyncio.wrap_future(self._loop.call("store_chunk", list(tokens)))
            return
        async with self._lock:
            await asyncio.get_running_loop().run_in_executor(None, self._guard, self._engine.store_chunk, list(tokens))

    def _pad_block(self, tokens: Sequence[int]) -> list[int]:
        bt = self._engine.cfg.block_tokens
        t = list(tokens)
        return t + [self._pad] * (-len(t) % bt)

    def _sampling(self, params: dict[str, Any]) -> dict[str, Any]:
        """Sampling and stopping fields of a request as the engines take them.  Greedy unless a
        positive temperature is asked for; an unseeded sampling request gets a fresh seed here, once,
        so that every tensor-parallel rank draws with the same one.  Generation stops at the model's
        end-of-sequence ids (unless ``ignore_eos``) and at the request's ``stop_token_ids``."""
        out: dict[str, Any] = {}
        stops = set(int(t) for t in (params.get("stop_token_ids") or []))
        if not params.get("ignore_eos"):
            stops.update(self.eos_token_ids)
        if stops:
            out["stop_token_ids"] = tuple(sorted(stops))
        t = float(params.get("temperature") or 0.0)
        if t > 0.0:
            seed = params.get("seed")
            out.update(temperature=t, seed=int(seed) if seed is not None else random.getrandbits(62))
            top_k, top_p = int(params.get("top_k") or 0), params.get("top_p")
            if top_k > 0:
                out["top_k"] = top_k
            if top_p is not None and 0.0 < float(top_p) < 1.0:
                out["top_p"] = float(top_p)
        return out

    def _generate(self, segments, query, max_new, on_token=None, sampling=None):
        eng = self._engine
        chunks = [self._pad_block(s) for s in segments if len(s)]
        if hasattr(eng, "generate"):
            kw = {"on_token": on_token} if on_token is not None else {}
            kw.update(sampling or {})
            req = eng.generate(chunks, list(query), max_new_tokens=max_new, **kw)
            return req.generated, req.context_len, getattr(req, "finish_reason", "") or "length"
        res = eng.run_request([], chunks, list(query))
        return [int(res.logits[-1].argmax())], res.total_tokens, "length"

    async def completion(self, tokens: list[int], gen_params: Optional[dict[str, Any]] = None,
                         segments: Optional[Sequence[Sequence[int]]] = None) -> dict[str, Any]:
        """``segments`` = cacheable token runs (document chunks) preceding the final query run;
        without them the whole prompt is computed."""
        params = gen_params or {}
        max_new = int(params.get("max_tokens", 256))
        if segments:
            *cached, query = segments
        else:
            cached, query = [], tokens
        sampling = self._sampling(params)
        if self._loop is not None:
            chunks = [self._pad_block(s) for s in cached if len(s)]
            req = await asyncio.wrap_future(self._loop.submit(chunks, query, max_new, **sampling))
            gen, prompt_len, why = req.generated, req.context_len, req.finish_reason or "length"
        else:
            async with self._lock:
                gen, prompt_len, why = await asyncio.get_running_loop().run_in_executor(
                    None, self._guard, self._generate, cached, query, max_new, None, sampling)
        return {
            "choices": [{"text": self._detok(gen), "token_ids": gen, "finish_reason": why}],
            "usage": {"prompt_tokens": prompt_len, "completion_tokens": len(gen)},
        }

    async def completion_stream(self, tokens: list[int], gen_params: Optional[dict[str, Any]] = None,
                                segments: Optional[Sequence[Sequence[int]]] = None):
        """Async generator over the request's tokens as the engine samples them: yields
        ``{"token_ids": [id], "text": piece}`` per token and a last item
        ``{"done": True, "usage": {...}}``.  The first item leaves as soon as the prefill step has
        ended, which is what makes the time to first token visible to an HTTP client."""
        params = gen_params or {}
        max_new = int(params.get("max_tokens", 256))
        if segments:
            *cached, query = segments
        else:
            cached, query = [], tokens
        sampling = self._sampling(params)
        loop = asyncio.get_running_loop()
        queue: asyncio.Queue = asyncio.Queue()
        push = lambda tok: loop.call_soon_threadsafe(queue.put_nowait, int(tok))  # noqa: E731
        async with (self._lock if self._loop is None else _NoLock()):
            if self._loop is not None:
                chunks = [self._pad_block(s) for s in cached if len(s)]

                ticket = self._loop.submit(chunks, query, max_new, on_token=push, **sampling)

                async def stepped():
                    req = await asyncio.wrap_future(ticket)
                    return req.generated, req.context_len, req.finish_reason or "length"

                fut = asyncio.ensure_future(stepped())
            else:
                fut = loop.run_in_executor(None, self._guard, self._generate, cached, query, max_new, push, sampling)
            fut.add_done_callback(lambda _f: queue.put_nowait(None))  # runs on the loop: after every token
            sent: list[int] = []
            text = ""
            try:
                while True:
                    tok = await queue.get()
                    if tok is None:
                        break
                    sent.append(tok)
                    # detokenise the whole run and send the new suffix: pieces of one token can change
                    # with what follows (byte-level merges)
                    full = self._detok(sent)
                    piece, text = (full[len(text):], full) if full.startswith(text) else (full, full)
                    yield {"token_ids": [tok], "text": piece}
            finally:
                # the consumer went away mid-stream (client disconnect closes this generator): take the
                # request out of the engine instead of generating the rest for nobody
                if self._loop is not None and not fut.done():
                    self._loop.cancel(ticket)
                    fut.cancel()
                elif not fut.done():
                    # one request at a time: the worker thread still owns the engine, so the lock must
                    # not be released before it is through (the tokens it still makes go nowhere)
                    try:
                        await asyncio.shield(fut)
                    except BaseException:
                        pass
            gen, prompt_len, why = await fut  # raises here if the engine failed
            if len(sent) < len(gen):  # an engine without token callbacks: everything at the end
                rest = gen[len(sent):]
                yield {"token_ids": rest, "text": self._detok(gen)[len(text):]}
        yield {"done": True, "finish_reason": why,
               "usage": {"prompt_tokens": prompt_len, "completion_tokens": len(gen)}}
