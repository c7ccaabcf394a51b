"""Split a token sequence into fixed-size, block-aligned chunks.

Capability parity: ``daser/service/chunker.py:33-105`` — chunks of
``block_tokens * chunk_blocks`` tokens (default 16 x 16 = 256), each keyed by the hash of its
own tokens; the trailing partial chunk is dropped from the cacheable set.  Added:
``tail`` returns the dropped remainder so the engine can still compute it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

from daser_b200.hashing import hash_tokens


@dataclass
class TokenChunk:
    index: int
    chunk_key: str
    tokens: list[int]


class Chunker:
    def __init__(self, block_tokens: int = 16, chunk_blocks: int = 16) -> None:
        if block_tokens <= 0 or chunk_blocks <= 0:
            raise ValueError("block_tokens and chunk_blocks must be positive")
        self._block_tokens = block_tokens
        self._chunk_blocks = chunk_blocks

    @property
    def block_tokens(self) -> int:
        return self._block_tokens

    @property
    def chunk_tokens(self) -> int:
        return self._block_tokens * self._chunk_blocks

    def chunk(self, tokens: Sequence[int]) -> list[TokenChunk]:
        n = self.chunk_tokens
        out = []
        for i in range(len(tokens) // n):
            part = list(tokens[i * n : (i + 1) * n])
            out.append(TokenChunk(i, hash_tokens(part), part))
        return out

    def tail(self, tokens: Sequence[int]) -> list[int]:
        n = self.chunk_tokens
        return list(tokens[(len(tokens) // n) * n :])
