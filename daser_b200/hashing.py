"""Chunk keys: XXH3-128 over little-endian int32 token ids.

The reference keeps three identical copies of this function that must stay in
lockstep (``daser/connector/daser_connector.py:41-57``,
``daser/retrieval/prefix.py:17-30``, ``daser/service/chunker.py:16-30``).  Here
there is one definition, and :func:`prefix_digests` produces the digest of
*every* block-aligned prefix in a single streaming pass, so a longest-prefix
lookup hashes O(n) bytes instead of the reference's O(n^2 / block).
The digests are bit-identical to hashing each prefix from scratch.
"""

from __future__ import annotations

from array import array
from typing import Sequence

import xxhash


def _token_bytes(tokens: Sequence[int]) -> bytes:
    buf = array("i", tokens)
    if buf.itemsize != 4:  # pragma: no cover - every supported ABI has 32-bit int
        raise RuntimeError("C int is not 32 bits on this platform")
    import sys

    if sys.byteorder != "little":  # pragma: no cover
        buf.byteswap()
    return buf.tobytes()


def hash_tokens(tokens: Sequence[int]) -> str:
    """32 hex characters identifying ``tokens`` (seed 0, canonical digest)."""
    return xxhash.xxh3_128(_token_bytes(tokens)).hexdigest()


def _native():
    from daser_b200.server import native_index

    return native_index if native_index.available() else None


def block_digests(tokens: Sequence[int], block_tokens: int) -> list[str]:
    """Digest of every aligned block ``tokens[i * b : (i + 1) * b]`` (anchor candidates of a scan)."""
    if block_tokens <= 0:
        raise ValueError("block_tokens must be positive")
    nat = _native()
    if nat is not None:
        return nat.block_digests(tokens, block_tokens)
    nblocks = len(tokens) // block_tokens
    raw = memoryview(_token_bytes(tokens[: nblocks * block_tokens]))
    step = block_tokens * 4
    return [xxhash.xxh3_128(raw[i * step : (i + 1) * step]).hexdigest() for i in range(nblocks)]


def window_digests(tokens: Sequence[int], block_tokens: int) -> list[str]:
    """Digest of ``tokens[i : i + b]`` at every token offset ``i`` (anchors at unaligned offsets)."""
    if block_tokens <= 0:
        raise ValueError("block_tokens must be positive")
    nat = _native()
    if nat is not None:
        return nat.window_digests(tokens, block_tokens)
    n = len(tokens) - block_tokens + 1
    if n <= 0:
        return []
    raw = memoryview(_token_bytes(tokens))
    step = block_tokens * 4
    return [xxhash.xxh3_128(raw[4 * i : 4 * i + step]).hexdigest() for i in range(n)]


def prefix_digests(tokens: Sequence[int], block_tokens: int) -> list[str]:
    """Digests of ``tokens[:b]`` for ``b = block_tokens, 2*block_tokens, ...``.

    Entry ``i`` equals ``hash_tokens(tokens[:(i + 1) * block_tokens])``.  One streaming pass, in
    the native library when it is built.
    """
    if block_tokens <= 0:
        raise ValueError("block_tokens must be positive")
    nblocks = len(tokens) // block_tokens
    if nblocks == 0:
        return []
    nat = _native()
    if nat is not None:
        return nat.prefix_digests(tokens, block_tokens)
    raw = memoryview(_token_bytes(tokens[: nblocks * block_tokens]))
    step = block_tokens * 4
    state = xxhash.xxh3_128()
    out = []
    for i in range(nblocks):
        state.update(raw[i * step : (i + 1) * step])
        out.append(state.hexdigest())
    return out
