"""The request record both engines schedule: what was asked, and what the engine filled in."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class RagRequest:
    chunks: list[list[int]]  # block-aligned token lists, concatenated in order (prefix first)
    query: list[int]
    max_new_tokens: int = 1
    req_id: str = ""
    arrival: float = 0.0
    # filled by the engine
    block_table: list[int] = field(default_factory=list)
    generated: list[int] = field(default_factory=list)
    context_len: int = 0
    ttft_ms: float = 0.0
    ttft_device_ms: float = 0.0
    first_token_time: float = 0.0  # time.perf_counter() when the first token was read back
    restored_chunks: int = 0
    restored_bytes: int = 0
    timings: dict = field(default_factory=dict)
    done: bool = False
    store_misses: bool = False  # write the KV of chunks that had to be computed (cold pass)
    # sampling: 0 = greedy; > 0 draws from softmax(logits / temperature), reproducibly from `seed`
    temperature: float = 0.0
    seed: int = 0
    top_k: int = 0  # with a temperature: sample among the k largest logits only (0 = all)
    top_p: float = 1.0  # ... and among the smallest set of them whose probability reaches p (1 = all)
    # set (with done) when the engine gave the request up without touching the others: it can never
    # fit the KV pool or the runner's buffers
    error: Optional[str] = None
    # generation also ends when one of these is sampled (end-of-sequence ids); the token stays in
    # `generated`, as in vLLM's token_ids
    stop_token_ids: tuple = ()
    finish_reason: str = ""  # "length" | "stop", set when generation ends
    # the chunks as the caller gave them, when the engine replaced a stored combination of them by
    # one chunk (composed-chunk reuse); empty otherwise
    asked: list = field(default_factory=list)

    def truncated(self) -> bool:
        return self.temperature > 0 and (self.top_k > 0 or self.top_p < 1.0)

    def finished(self) -> bool:
        """Has the token just appended ended the generation?  Records why."""
        if self.generated and self.stop_token_ids and self.generated[-1] in self.stop_token_ids:
            self.finish_reason = "stop"
            return True
        if len(self.generated) >= self.max_new_tokens:
            self.finish_reason = "length"
            return True
        return False

    def blocks_needed(self, block_tokens: int) -> int:
        """KV blocks of the whole request, generation included (reserved up front, so that a running
        request can never be starved of blocks by later arrivals)."""
        total = sum(len(c) for c in self.chunks) + len(self.query) + self.max_new_tokens
        return -(-total // block_tokens)

    def step_seed(self) -> int:
        """The seed of the token about to be sampled (one stream of noise per request and step)."""
        return (self.seed * 1_000_003 + len(self.generated) + 1) & 0x7FFFFFFFFFFFFFFF
