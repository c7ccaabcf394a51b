"""ctypes binding of the native token index (``server/csrc/token_index.cc``).

:func:`available` is False when the library was not built or the system has no libxxhash; the
callers (``hashing.py``, ``retrieval/prefix.py``) then use the pure-Python path, which produces
the same digests through the ``xxhash`` wheel.
"""

from __future__ import annotations

import ctypes as C
from array import array
from pathlib import Path
from typing import Optional, Sequence

_LIB_PATH = Path(__file__).resolve().parent / "libdaser_index.so"
_lib: Optional[C.CDLL] = None
_raw: Optional[C.CDLL] = None  # the library whether or not libxxhash was found (the lookup server needs none)
_checked = False


def _load() -> Optional[C.CDLL]:
    global _lib, _raw, _checked
    if _checked:
        return _lib
    _checked = True
    if not _LIB_PATH.exists():
        return None
    try:
        lib = C.CDLL(str(_LIB_PATH))
    except OSError:
        return None
    p, i64, i32, u64 = C.c_void_p, C.c_int64, C.c_int32, C.c_uint64
    lib.daser_index_available.restype = C.c_int
    lib.daser_hash_tokens.argtypes = [p, i64, p]
    for fn in (lib.daser_prefix_digests, lib.daser_block_digests, lib.daser_window_digests):
        fn.argtypes, fn.restype = [p, i64, i32, p], i64
    lib.daser_table_new.argtypes, lib.daser_table_new.restype = [i64], p
    lib.daser_table_free.argtypes = [p]
    lib.daser_table_size.argtypes, lib.daser_table_size.restype = [p], i64
    lib.daser_table_put.argtypes = [p, u64, p, i64]
    lib.daser_table_del.argtypes = [p, u64, p]
    lib.daser_table_get.argtypes, lib.daser_table_get.restype = [p, u64, p, i64], i64
    lib.daser_table_longest_prefix.argtypes = [p, u64, p, i64, i32, i64, C.POINTER(i64)]
    lib.daser_table_longest_prefix.restype = i64
    lib.daser_table_scan_blocks.argtypes, lib.daser_table_scan_blocks.restype = [p, u64, p, i64, i32, p, p, i64], i64
    if hasattr(lib, "daser_fast_start"):
        cs = C.c_char_p
        lib.daser_fast_start.argtypes, lib.daser_fast_start.restype = [cs, i64], p
        lib.daser_fast_stop.argtypes = [p]
        lib.daser_fast_put.argtypes = [p, cs, cs, i64, i64, i64, i64]
        lib.daser_fast_del.argtypes = [p, cs]
        lib.daser_fast_clear.argtypes = [p]
        lib.daser_fast_stats.argtypes = [p, p]
        _raw = lib
    if lib.daser_index_available() != 1:
        return None
    _lib = lib
    return _lib


def available() -> bool:
    return _load() is not None


def _tokens(tokens: Sequence[int]):
    buf = tokens if isinstance(tokens, array) and tokens.typecode == "i" else array("i", tokens)
    addr, n = buf.buffer_info()
    return buf, C.c_void_p(addr), n


def hash_tokens(tokens: Sequence[int]) -> str:
    buf, ptr, n = _tokens(tokens)
    out = C.create_string_buffer(16)
    if _load().daser_hash_tokens(ptr, n, out) != 0:
        raise RuntimeError("native hash failed")
    return out.raw.hex()


def _digests(fn, tokens: Sequence[int], block: int) -> list[str]:
    buf, ptr, n = _tokens(tokens)
    nb = n // block
    if nb == 0:
        return []
    out = C.create_string_buffer(16 * nb)
    if fn(ptr, n, block, out) != nb:
        raise RuntimeError("native digest pass failed")
    raw = out.raw
    return [raw[16 * i : 16 * i + 16].hex() for i in range(nb)]


def prefix_digests(tokens: Sequence[int], block: int) -> list[str]:
    return _digests(_load().daser_prefix_digests, tokens, block)


def block_digests(tokens: Sequence[int], block: int) -> list[str]:
    return _digests(_load().daser_block_digests, tokens, block)


def window_digests(tokens: Sequence[int], block: int) -> list[str]:
    """Digest of ``tokens[i : i + block]`` for every offset ``i``."""
    buf, ptr, n = _tokens(tokens)
    nw = n - block + 1 if n >= block else 0
    if nw == 0:
        return []
    out = C.create_string_buffer(16 * nw)
    if _load().daser_window_digests(ptr, n, block, out) != nw:
        raise RuntimeError("native digest pass failed")
    raw = out.raw
    return [raw[16 * i : 16 * i + 16].hex() for i in range(nw)]


class DigestTable:
    """(model tag, 128-bit digest) -> int64, with longest-prefix and anchor-scan queries in one call."""

    MISSING = -1

    def __init__(self, capacity_hint: int = 1024) -> None:
        self._lib = _load()
        if self._lib is None:
            raise RuntimeError("native index unavailable")
        self._t = self._lib.daser_table_new(capacity_hint)

    def __del__(self) -> None:
        t, self._t = getattr(self, "_t", None), None
        if t and self._lib is not None:
            self._lib.daser_table_free(t)

    def __len__(self) -> int:
        return int(self._lib.daser_table_size(self._t))

    def put(self, tag: int, digest_hex: str, value: int) -> None:
        self._lib.daser_table_put(self._t, tag, bytes.fromhex(digest_hex), value)

    def delete(self, tag: int, digest_hex: str) -> bool:
        return self._lib.daser_table_del(self._t, tag, bytes.fromhex(digest_hex)) == 1

    def get(self, tag: int, digest_hex: str) -> int:
        return int(self._lib.daser_table_get(self._t, tag, bytes.fromhex(digest_hex), self.MISSING))

    def longest_prefix(self, tag: int, tokens: Sequence[int], block: int) -> tuple[int, int]:
        """(value, matched tokens) of the longest stored block-aligned prefix, or (MISSING, 0)."""
        buf, ptr, n = _tokens(tokens)
        matched = C.c_int64(0)
        v = self._lib.daser_table_longest_prefix(self._t, tag, ptr, n, block, self.MISSING, C.byref(matched))
        return int(v), int(matched.value)

    def scan_blocks(self, tag: int, tokens: Sequence[int], block: int) -> list[tuple[int, int]]:
        """(block index, value) of every aligned block of ``tokens`` that is a key of the table."""
        buf, ptr, n = _tokens(tokens)
        cap = max(1, n // max(block, 1))
        idx = (C.c_int64 * cap)()
        val = (C.c_int64 * cap)()
        hits = int(self._lib.daser_table_scan_blocks(self._t, tag, ptr, n, block, idx, val, cap))
        return [(int(idx[i]), int(val[i])) for i in range(min(hits, cap))]


class FastLookupServer:
    """The native thread that answers ``lookup_chunks {keys}`` on a socket of its own
    (``server/csrc/fast_lookup.cc``).  The Python server keeps its records in step: :meth:`put`
    when a chunk becomes visible, :meth:`delete` when it is evicted or aborted."""

    def __init__(self, socket_path: str, slot_size: int) -> None:
        _load()
        if _raw is None:
            raise RuntimeError("the native library was not built")
        self.socket_path = socket_path
        self._lib = _raw
        self._h = self._lib.daser_fast_start(socket_path.encode(), slot_size)
        if not self._h:
            raise OSError(f"cannot listen on {socket_path}")

    @staticmethod
    def supported() -> bool:
        _load()
        return _raw is not None

    def put(self, key: str, model_id: str, start_slot: int, num_slots: int, token_count: int, pos_offset: int) -> None:
        if self._h:
            self._lib.daser_fast_put(self._h, key.encode(), model_id.encode(), start_slot, num_slots, token_count,
                                     pos_offset)

    def delete(self, key: str) -> None:
        if self._h:
            self._lib.daser_fast_del(self._h, key.encode())

    def clear(self) -> None:
        if self._h:
            self._lib.daser_fast_clear(self._h)

    def stats(self) -> dict[str, int]:
        out = (C.c_int64 * 5)()
        if self._h:
            self._lib.daser_fast_stats(self._h, out)
        return dict(zip(("records", "calls", "hits", "misses", "refused"), (int(v) for v in out)))

    def stop(self) -> None:
        if self._h:
            self._lib.daser_fast_stop(self._h)
            self._h = None

    def __del__(self) -> None:
        try:
            self.stop()
        except Exception:
            pass
