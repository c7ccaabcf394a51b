"""REST front end.

Capability parity: ``daser/service/http_api.py:22-271`` — ``ServiceConfig``, the pydantic
bodies, ``_tokenize`` (no special tokens) and ``build_service_app`` with the six routes:
``GET /health``, ``POST /documents`` (201), ``GET /documents``, ``GET /documents/{id}``,
``DELETE /documents/{id}``, ``POST /infer``, with the same status codes (400 short document
or empty ids, 404 unknown document, 409 document without tokens, 502 engine or IPC failure).

Differences:

* the engine is anything with ``prefill / completion / health`` — a remote vLLM or the
  in-process native engine;
* ``/infer`` hands the engine the prompt *segments* (system prompt, each document chunk,
  separators, task), so cached chunks are restored at their offsets.  In the reference the
  uploaded chunks can never be hit by ``/infer`` because only whole-prompt prefixes are
  looked up;
* chunk prefills of an upload run concurrently (bounded) instead of one by one;
* ``GET /metrics`` exposes the counters in Prometheus text format;
* ``tokenizer="byte"`` selects a built-in UTF-8 byte tokenizer so the service runs with no
  model files.
"""

from __future__ import annotations

import asyncio
import time
import uuid
from contextlib import asynccontextmanager
from dataclasses import dataclass
from typing import Any, Optional

from fastapi import FastAPI, HTTPException
from fastapi.responses import PlainTextResponse
from pydantic import BaseModel, Field

from daser_b200 import metrics
from daser_b200.connector.ipc_client import IPCClientAsync
from daser_b200.logging import init_logger
from daser_b200.service.chunker import Chunker

logger = init_logger(__name__)


@dataclass
class ServiceConfig:
    vllm_base_url: str
    model: str
    tokenizer: str
    socket_path: str
    block_tokens: int = 16
    chunk_blocks: int = 16
    system_prompt: str = "You are a helpful assistant answering questions using the following documents.\n\n"
    doc_separator: str = "\n\n---\n\n"
    task_separator: str = "\n\n---\nTask: "
    upload_concurrency: int = 4


class UploadRequest(BaseModel):
    title: str = Field(..., description="Display title for the document")
    text: str = Field(..., description="Raw document text")


class InferRequest(BaseModel):
    doc_ids: list[str] = Field(..., description="Doc IDs to include in the prompt")
    task: str = Field(..., description="User task / question appended after documents")
    gen_params: Optional[dict[str, Any]] = Field(default=None, description="OpenAI-style generation parameters")


class ByteTokenizer:
    """UTF-8 bytes as token ids (offset by 3 to leave room for pad/bos/eos)."""

    def __call__(self, text: str, add_special_tokens: bool = False) -> dict[str, list[int]]:
        return {"input_ids": [b + 3 for b in text.encode("utf-8")]}

    def decode(self, ids) -> str:
        return bytes(max(0, min(255, int(i) - 3)) for i in ids).decode("utf-8", errors="replace")


def load_tokenizer(name: str):
    if name == "byte":
        return ByteTokenizer()
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(name)


def _tokenize(tokenizer, text: str) -> list[int]:
    return list(tokenizer(text, add_special_tokens=False)["input_ids"])


def build_service_app(cfg: ServiceConfig, engine_client: Any = None, tokenizer: Any = None) -> FastAPI:
    tok = tokenizer or load_tokenizer(cfg.tokenizer)
    chunker = Chunker(cfg.block_tokens, cfg.chunk_blocks)
    ipc = IPCClientAsync(cfg.socket_path)
    if engine_client is None:
        from daser_b200.service.vllm_client import VLLMClient

        engine_client = VLLMClient(cfg.vllm_base_url, cfg.model)
    engine = engine_client

    @asynccontextmanager
    async def lifespan(_app: FastAPI):
        yield
        await engine.close()
        await ipc.close()

    app = FastAPI(title="daser_b200 service", version="0.1.0", lifespan=lifespan)

    @app.get("/health")
    async def health() -> dict[str, Any]:
        ok = await engine.health()
        return {"status": "ok" if ok else "degraded", "vllm": ok}

    @app.get("/metrics", response_class=PlainTextResponse)
    async def prometheus() -> str:
        return metrics.prometheus_text()

    @app.post("/documents", status_code=201)
    async def upload_document(req: UploadRequest) -> dict[str, Any]:
        tokens = _tokenize(tok, req.text)
        chunks = chunker.chunk(tokens)
        if not chunks:
            raise HTTPException(400, f"document shorter than one chunk ({chunker.chunk_tokens} tokens)")
        t0 = time.time()
        sem = asyncio.Semaphore(max(1, cfg.upload_concurrency))

        async def one(chunk):
            async with sem:
                await engine.prefill(chunk.tokens)

        try:
            await asyncio.gather(*(one(c) for c in chunks))
        except Exception as exc:
            logger.error("[SERVICE] prefill failed: %r", exc)
            raise HTTPException(502, f"engine prefill failed: {exc}") from exc
        prefill_ms = (time.time() - t0) * 1e3
        metrics.observe("service.prefill_ms", prefill_ms)
        doc_id = uuid.uuid4().hex
        try:
            reply = await ipc.register_doc(doc_id, req.title, [c.chunk_key for c in chunks], len(tokens), tokens)
        except RuntimeError as exc:
            raise HTTPException(502, f"control plane error: {exc}") from exc
        return {"doc_id": doc_id, "status": "ready", "chunk_count": len(chunks),
                "chunk_count_cached": reply.get("chunk_count_cached", 0), "prefill_ms": round(prefill_ms, 1)}

    @app.get("/documents")
    async def list_documents() -> list[dict[str, Any]]:
        try:
            return await ipc.list_docs()
        except RuntimeError as exc:
            raise HTTPException(502, str(exc)) from exc

    @app.get("/documents/{doc_id}")
    async def get_document(doc_id: str) -> dict[str, Any]:
        try:
            doc = await ipc.get_doc(doc_id)
        except RuntimeError as exc:
            raise HTTPException(404, f"unknown document {doc_id}") from exc
        doc.pop("tokens", None)
        return doc

    @app.delete("/documents/{doc_id}")
    async def delete_document(doc_id: str) -> dict[str, Any]:
        try:
            reply = await ipc.evict_doc(doc_id)
        except RuntimeError as exc:
            raise HTTPException(404, f"unknown document {doc_id}") from exc
        return {"ok": True, "chunks_evicted": reply.get("chunks_evicted", 0)}

    @app.post("/infer")
    async def infer(req: InferRequest) -> dict[str, Any]:
        if not req.doc_ids:
            raise HTTPException(400, "doc_ids must not be empty")
        segments: list[list[int]] = [_tokenize(tok, cfg.system_prompt)]
        sep = _tokenize(tok, cfg.doc_separator)
        for i, doc_id in enumerate(req.doc_ids):
            try:
                doc = await ipc.get_doc(doc_id)
            except RuntimeError as exc:
                raise HTTPException(404, f"unknown document {doc_id}") from exc
            if not doc.get("tokens"):
                raise HTTPException(409, f"document {doc_id} has no stored tokens")
            if i:
                segments.append(sep)
            doc_tokens = list(doc["tokens"])
            segments.extend(c.tokens for c in chunker.chunk(doc_tokens))
            tail = chunker.tail(doc_tokens)
            if tail:
                segments.append(tail)
        segments.append(_tokenize(tok, cfg.task_separator) + _tokenize(tok, req.task))
        prompt = [t for seg in segments for t in seg]
        t0 = time.time()
        try:
            reply = await engine.completion(prompt, req.gen_params, segments=segments)
        except Exception as exc:
            logger.error("[SERVICE] completion failed: %r", exc)
            raise HTTPException(502, f"engine completion failed: {exc}") from exc
        latency_ms = (time.time() - t0) * 1e3
        metrics.observe("service.infer_ms", latency_ms)
        usage = reply.get("usage", {})
        choice = (reply.get("choices") or [{}])[0]
        return {"text": choice.get("text", ""), "prompt_tokens": usage.get("prompt_tokens", len(prompt)),
                "completion_tokens": usage.get("completion_tokens", 0), "latency_ms": round(latency_ms, 1)}

    return app
