"""Chunk-level retrieval: find cached chunks anywhere inside a prompt.

No counterpart in the reference, whose only index matches prompt *prefixes*;
a chunk uploaded through its service (keyed by the hash of the chunk's own
tokens) can therefore never be hit by an ``/infer`` prompt that starts with a
system prompt (``daser/service/http_api.py:138-146,221-245`` against
``daser/retrieval/prefix.py:63-72``).  This index answers two questions:

* ``lookup_keys`` — batched exact lookup by ``chunk_key``; the caller already
  knows which document chunks it concatenated (the RAG case).
* ``scan`` — given only the prompt tokens, find every stored chunk that
  appears at a block-aligned offset.  Each stored chunk registers the digest
  of its first block as an anchor; a scan hashes each block of the prompt once
  and verifies candidates by hashing the full span, so the cost is linear in
  the prompt plus the verified spans.

``lookup`` (the ABC method) falls back to prefix semantics so this class can
stand wherever a :class:`PrefixHashIndex` does.
"""

from __future__ import annotations

from dataclasses import dataclass

from daser_b200.hashing import block_digests, hash_tokens, window_digests
from daser_b200.retrieval.prefix import PrefixHashIndex
from daser_b200.server.metadata_store import ChunkMeta


@dataclass
class ChunkHit:
    """A stored chunk found at token offset ``offset`` of the query."""

    meta: ChunkMeta
    offset: int


class ChunkOffsetIndex(PrefixHashIndex):
    def __init__(self, block_tokens: int = 16, native: bool | None = None) -> None:
        super().__init__(block_tokens, native)
        self._anchors: dict[str, set[str]] = {}
        self._anchor_of: dict[str, str] = {}

    def register_anchor(self, chunk_key: str, first_block_digest: str) -> None:
        """Associate a committed chunk with the digest of its first block."""
        if chunk_key not in self._by_key:
            return
        self._anchors.setdefault(first_block_digest, set()).add(chunk_key)
        self._anchor_of[chunk_key] = first_block_digest

    def lookup_keys(self, keys: list[str], model_id: str) -> list[ChunkMeta | None]:
        out: list[ChunkMeta | None] = []
        for key in keys:
            meta = self._by_key.get(key)
            out.append(meta if meta is not None and meta.model_id == model_id else None)
        return out

    def scan(self, tokens: list[int], model_id: str, any_offset: bool = False) -> list[ChunkHit]:
        """Non-overlapping stored chunks, left to right: at block-aligned offsets, or with
        ``any_offset`` at every token offset (a caller that pads what precedes a hit can then
        still place the chunk on a block boundary)."""
        bt = self._block_tokens
        hits: list[ChunkHit] = []
        pos = 0
        n = len(tokens)
        if not self._anchors:
            return hits
        # every candidate first block is hashed once, in one pass (native when built)
        step = 1 if any_offset else bt
        anchors = window_digests(tokens, bt) if any_offset else block_digests(tokens, bt)
        while pos + bt <= n:
            best: ChunkMeta | None = None
            keys = self._anchors.get(anchors[pos // step])
            if keys:
                for key in keys:
                    meta = self._by_key.get(key)
                    if meta is None or meta.model_id != model_id:
                        continue
                    span = meta.token_count
                    if pos + span > n or (best and span <= best.token_count):
                        continue
                    if hash_tokens(tokens[pos : pos + span]) == key:
                        best = meta
            if best is not None:
                hits.append(ChunkHit(best, pos))
                pos += best.token_count if any_offset else -(-best.token_count // bt) * bt
            else:
                pos += step
        return hits

    def _forget(self, chunk_key: str) -> None:
        anchor = self._anchor_of.pop(chunk_key, None)
        if anchor is not None:
            keys = self._anchors.get(anchor)
            if keys is not None:
                keys.discard(chunk_key)
                if not keys:
                    del self._anchors[anchor]

    async def remove(self, chunk_key: str) -> None:
        self._forget(chunk_key)
        await super().remove(chunk_key)

    def discard(self, chunk_key: str) -> None:
        self._forget(chunk_key)
        super().discard(chunk_key)
