"""A minimal OpenAI-compatible completions endpoint in front of the in-process engine.

The reference's service (and its benchmarks) drive a remote stock vLLM through
``POST /v1/completions`` with token-id prompts (``daser/service/vllm_client.py:62-126``).  With
these routes mounted, the native engine answers the same calls, so that client (or this
repository's :class:`~daser_b200.service.vllm_client.VLLMClient`) can point at it unchanged:

* ``POST /v1/completions``  ``{"model", "prompt": [token ids] | "text", "max_tokens", ...}``
* ``POST /v1/chat/completions``  ``{"model", "messages": [{"role", "content"}], "max_tokens", ...}`` (the
  tokenizer's chat template when it has one)
* ``GET  /v1/models``, ``GET /health``

A request with ``max_tokens == 1`` is what the reference's service uses as "prefill this chunk so
that the cache holds it" (vLLM's connector stores the KV of every prompt it has not seen); the same
side effect happens here: when the prompt's block-aligned prefix is not stored yet, it is stored as
a chunk keyed by the hash of its tokens, which is the key the reference's chunker registers.

Cache reuse needs no cooperation from the caller: the prompt's token ids are scanned against the
control plane (``lookup_chunks`` with tokens: every stored chunk that appears at a block-aligned
offset), the prompt is cut at the hits, and the pieces go to the engine as segments: hits are
restored (keys re-rotated to their new positions), the gaps and the tail are computed.  Sampling is
greedy by default (``temperature`` 0); a positive ``temperature`` draws from the softmax, reproducibly
when ``seed`` is given, optionally truncated by ``top_k`` / ``top_p``.  Penalties are accepted and
ignored; ``n`` or
``best_of`` above 1, ``logprobs``, ``echo`` and ``stop`` strings are refused (400) rather than silently
dropped (``stop_token_ids`` work).

``"stream": true`` answers with server-sent events, one per sampled token (vLLM's shape), so a
client sees the first token when the prefill step ends rather than when the request does.
"""

from __future__ import annotations

import json
import time
import uuid
from typing import Any, Optional, Sequence

from fastapi import FastAPI, HTTPException
from fastapi.responses import StreamingResponse
from pydantic import BaseModel

from daser_b200 import metrics
from daser_b200.connector.ipc_client import IPCClientAsync
from daser_b200.logging import init_logger

logger = init_logger(__name__)


class CompletionRequest(BaseModel):
    model: Optional[str] = None
    prompt: Any
    max_tokens: int = 16
    temperature: float = 0.0
    seed: Optional[int] = None
    stream: bool = False

    model_config = {"extra": "allow"}


class ChatRequest(BaseModel):
    model: Optional[str] = None
    messages: list[dict[str, Any]]
    max_tokens: int = 16
    temperature: float = 0.0
    seed: Optional[int] = None
    stream: bool = False

    model_config = {"extra": "allow"}


def chat_prompt_tokens(tokenizer: Any, messages: list[dict[str, Any]]) -> list[int]:
    """Token ids of a chat: the tokenizer's own template when it has one (``transformers``
    tokenizers of chat models), else ``role: content`` lines and an open assistant line."""
    if hasattr(tokenizer, "apply_chat_template") and getattr(tokenizer, "chat_template", None):
        out = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
        ids = out["input_ids"] if isinstance(out, dict) else out
        return [int(t) for t in ids]
    text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in messages) + "assistant:"
    return list(tokenizer(text, add_special_tokens=False)["input_ids"])


def split_at_hits(tokens: Sequence[int], hits: Sequence[dict[str, Any]], block_tokens: int,
                  aligned_only: bool = False) -> list[list[int]]:
    """Cut ``tokens`` into segments at the stored chunks found in it.

    Every segment but the last is a stored chunk or the gap before one; the last one is the
    query the engine computes and is never empty.  The engine client pads every segment but the
    last to a block boundary, which is what puts a chunk found at an odd offset back on one (at
    the price of pad tokens in the context); ``aligned_only`` keeps only hits that need no padding.
    """
    segments: list[list[int]] = []
    pos = 0
    n = len(tokens)
    for hit in sorted(hits, key=lambda h: h["offset"]):
        off, count = int(hit["offset"]), int(hit["token_count"])
        if off < pos or off + count >= n or (aligned_only and off % block_tokens):
            continue  # overlaps the previous hit, or would leave no token to compute
        if off > pos:
            segments.append(list(tokens[pos:off]))
        segments.append(list(tokens[off : off + count]))
        pos = off + count
    segments.append(list(tokens[pos:]))
    return segments


def _gen_params(req: Any) -> dict[str, Any]:
    params: dict[str, Any] = {"max_tokens": req.max_tokens, "temperature": req.temperature}
    if req.seed is not None:
        params["seed"] = req.seed
    extra = getattr(req, "model_extra", None) or {}  # vLLM's extensions, passed as plain fields
    for name in ("stop_token_ids", "ignore_eos", "top_k", "top_p"):
        if extra.get(name) is not None:
            params[name] = extra[name]
    return params


def _choice(chat: bool, text: str, token_ids: Any, finish: Optional[str], delta: bool) -> dict[str, Any]:
    """One ``choices`` entry in the completions or the chat shape (``delta`` in stream events)."""
    if not chat:
        return {"index": 0, "text": text, "token_ids": token_ids, "logprobs": None, "finish_reason": finish}
    body = {"role": "assistant", "content": text}
    return {"index": 0, ("delta" if delta else "message"): body, "token_ids": token_ids, "logprobs": None,
            "finish_reason": finish}


async def _sse(engine_client: Any, req: Any, tokens: list[int], segments: list[list[int]],
               model_name: str, t0: float, chat: bool = False):
    """Server-sent events in vLLM's shape: one ``text_completion`` object per token, a last one with
    ``finish_reason`` and ``usage``, then ``data: [DONE]``.  The first event is the time to first
    token as an HTTP client sees it (recorded as ``service.stream_ttft_ms``)."""
    rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex
    base = {"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "created": int(t0),
            "model": req.model or model_name}
    first = True
    try:
        async for item in engine_client.completion_stream(tokens, _gen_params(req), segments=segments):
            if item.get("done"):
                usage = item["usage"]
                n_out = int(usage.get("completion_tokens", 0))
                last = dict(base, choices=[_choice(chat, "", [], item.get("finish_reason", "length"), True)],
                            usage={"prompt_tokens": len(tokens), "completion_tokens": n_out,
                                   "total_tokens": len(tokens) + n_out})
                yield f"data: {json.dumps(last)}\n\n"
                break
            if first:
                metrics.observe("service.stream_ttft_ms", (time.time() - t0) * 1e3)
                first = False
            event = dict(base, choices=[_choice(chat, item["text"], item["token_ids"], None, True)])
            yield f"data: {json.dumps(event)}\n\n"
    except Exception as exc:  # the status line has gone out already: report in-band, as vLLM does
        logger.warning("[SERVICE] streamed completion failed: %s", exc)
        yield f"data: {json.dumps({'error': {'message': f'engine failed: {exc}', 'code': 502}})}\n\n"
    metrics.observe("service.completion_ms", (time.time() - t0) * 1e3)
    yield "data: [DONE]\n\n"


def mount_openai_routes(app: FastAPI, engine_client: Any, tokenizer: Any, socket_path: str, model_name: str,
                        model_id: str = "default", block_tokens: int = 16) -> None:
    ipc = IPCClientAsync(socket_path)

    @app.get("/v1/models")
    async def models() -> dict[str, Any]:
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "daser_b200"}]}

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest) -> Any:
        prompt = req.prompt
        if isinstance(prompt, str):
            tokens = list(tokenizer(prompt, add_special_tokens=False)["input_ids"])
        elif isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            tokens = list(prompt)
        elif isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], list):
            tokens = [int(t) for t in prompt[0]]
        elif isinstance(prompt, list) and len(prompt) > 1 and all(isinstance(p, (str, list)) for p in prompt):
            # several prompts in one call (vLLM's batch form): served side by side, which the engine
            # loop turns into shared steps; one choice per prompt, in order
            if req.stream:
                raise HTTPException(400, "streaming takes one prompt per request")
            import asyncio

            singles = [req.model_copy(update={"prompt": p if isinstance(p, str) else [int(t) for t in p]})
                       for p in prompt]
            parts = await asyncio.gather(*(completions(r) for r in singles))
            usage = {k: sum(p["usage"][k] for p in parts) for k in ("prompt_tokens", "completion_tokens", "total_tokens")}
            return dict(parts[0], choices=[dict(p["choices"][0], index=i) for i, p in enumerate(parts)], usage=usage)
        else:
            raise HTTPException(400, "prompt must be a string or a list of token ids")
        return await serve(req, tokens, chat=False)

    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatRequest) -> Any:
        if not req.messages:
            raise HTTPException(400, "messages must not be empty")
        return await serve(req, chat_prompt_tokens(tokenizer, req.messages), chat=True)

    async def serve(req: Any, tokens: list[int], chat: bool) -> Any:
        extra = getattr(req, "model_extra", None) or {}
        for name, limit in (("n", 1), ("best_of", 1)):
            if extra.get(name) not in (None, limit):
                raise HTTPException(400, f"{name} other than {limit} is not supported")
        if extra.get("logprobs") or extra.get("top_logprobs") or extra.get("echo"):
            raise HTTPException(400, "logprobs / echo are not supported")
        if extra.get("stop"):
            raise HTTPException(400, "stop strings are not supported (stop_token_ids are)")
        if not tokens:
            raise HTTPException(400, "empty prompt")
        if req.max_tokens < 1:
            raise HTTPException(400, "max_tokens must be at least 1")  # as vLLM
        t0 = time.time()
        try:
            # token ids as one packed int32 field (a control plane of this package takes them; a list
            # of n msgpack integers costs several times as much on both ends)
            from array import array

            reply = await ipc.call({"op": "lookup_chunks", "tokens_bin": array("i", tokens).tobytes(),
                                    "model_id": model_id, "any_offset": True})
            hits = reply.get("hits", [])
        except RuntimeError as exc:  # the control plane is optional for correctness: compute everything
            logger.warning("[SERVICE] scan failed (%s): computing the whole prompt", exc)
            hits = []
        segments = split_at_hits(tokens, hits, block_tokens)
        if req.stream:
            if not hasattr(engine_client, "completion_stream"):
                raise HTTPException(400, "streaming is not supported by this engine client")
            return StreamingResponse(_sse(engine_client, req, tokens, segments, model_name, t0, chat),
                                     media_type="text/event-stream")
        try:
            out = await engine_client.completion(tokens, _gen_params(req), segments=segments)
            aligned = len(tokens) // block_tokens * block_tokens
            covered = any(int(h["offset"]) == 0 and int(h["token_count"]) >= aligned for h in hits)
            if req.max_tokens == 1 and aligned and not covered:
                await engine_client.prefill(tokens[:aligned])  # a prefill request leaves its KV in the store
                metrics.inc("service.completion_stores")
        except MemoryError as exc:  # the request can never fit the KV pool: the caller's problem, as in vLLM
            raise HTTPException(400, f"request too large: {exc}") from exc
        except RuntimeError as exc:
            if type(exc).__name__ == "QueueFull":  # back-pressure of the engine loop
                raise HTTPException(429, str(exc)) from exc
            raise HTTPException(502, f"engine failed: {exc}") from exc
        except Exception as exc:
            raise HTTPException(502, f"engine failed: {exc}") from exc
        metrics.observe("service.completion_ms", (time.time() - t0) * 1e3)
        metrics.inc("service.completion_hits", len(segments) - 1 if hits else 0)
        choice = out["choices"][0]
        usage = out.get("usage", {})
        n_out = int(usage.get("completion_tokens", len(choice.get("token_ids", []))))
        return {
            "id": ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex,
            "object": "chat.completion" if chat else "text_completion", "created": int(t0),
            "model": req.model or model_name,
            "choices": [_choice(chat, choice.get("text", ""), choice.get("token_ids"),
                                choice.get("finish_reason", "length"), False)],
            "usage": {"prompt_tokens": len(tokens), "completion_tokens": n_out, "total_tokens": len(tokens) + n_out},
        }
