"""Python face of the native storage engine (``io/csrc/io_engine.cc``)."""

from __future__ import annotations

import ctypes as C
import enum
import os
from pathlib import Path
from typing import Optional, Sequence

_LIB_PATH = Path(__file__).resolve().parent / "libdaser_io.so"
_lib: Optional[C.CDLL] = None


class IOBackend(enum.Enum):
    AUTO = 0
    GDS = 1
    IO_URING = 2
    POSIX = 3


class IOTimeout(TimeoutError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            from daser_b200.ops.build import build_io

            build_io()
        L = C.CDLL(str(_LIB_PATH))
        L.daser_io_open.restype = C.c_void_p
        L.daser_io_open.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int,
                                    C.POINTER(C.c_int)]
        L.daser_io_backend.argtypes = [C.c_void_p]
        L.daser_io_file_size.restype = C.c_int64
        L.daser_io_file_size.argtypes = [C.c_void_p]
        L.daser_io_submit.restype = C.c_int64
        L.daser_io_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64]
        L.daser_io_submit_strided.restype = C.c_int64
        L.daser_io_submit_strided.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                              C.c_int, C.c_int64]
        L.daser_io_wait.argtypes = [C.c_void_p, C.c_int64, C.c_int]
        L.daser_io_poll.argtypes = [C.c_void_p, C.c_int64]
        L.daser_io_close.argtypes = [C.c_void_p]
        L.daser_io_preallocate.argtypes = [C.c_char_p, C.c_int64]
        L.daser_io_inject.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64]
        L.daser_io_stats.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        L.daser_io_register_buffers.restype = C.c_int64
        L.daser_io_register_buffers.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int]
        L.daser_io_fixed_pieces.restype = C.c_int64
        L.daser_io_fixed_pieces.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def preallocate(path: str, size: int) -> None:
    """Create or extend ``path`` to ``size`` bytes with ``posix_fallocate`` (no user-space zeros).

    The reference zero-fills a new store by writing a Python ``bytes`` of the whole size
    (``daser/connector/daser_connector.py:416-427``).
    """
    rc = lib().daser_io_preallocate(path.encode(), size)
    if rc < 0:
        raise OSError(-rc, os.strerror(-rc), path)


class IOEngine:
    """One open store file.  ``submit_*`` return tickets; ``wait`` blocks (GIL released)."""

    def __init__(self, path: str, backend: IOBackend = IOBackend.AUTO, device: Optional[int] = None,
                 queue_depth: int = 64, nthreads: int = 4) -> None:
        err = C.create_string_buffer(256)
        err_no = C.c_int(0)
        self._h = lib().daser_io_open(path.encode(), backend.value, 0 if device is None else device + 1,
                                      queue_depth, nthreads, err, 256, C.byref(err_no))
        if not self._h:
            if err_no.value == 2:
                raise FileNotFoundError(path)
            raise OSError(err_no.value, err.value.decode() or "daser_io_open failed", path)
        self.path = path
        self.backend = IOBackend(lib().daser_io_backend(self._h))

    @property
    def file_size(self) -> int:
        return lib().daser_io_file_size(self._h)

    def _submit(self, write: bool, ptr: int, device: bool, offset: int, nbytes: int) -> int:
        if self._h is None:
            raise ValueError("engine is closed")
        t = lib().daser_io_submit(self._h, int(write), C.c_void_p(ptr), int(device), offset, nbytes)
        if t < 0:
            raise OSError(-t, os.strerror(-t))
        return t

    def submit_read(self, ptr: int, offset: int, nbytes: int, device: bool = False) -> int:
        return self._submit(False, ptr, device, offset, nbytes)

    def submit_write(self, ptr: int, offset: int, nbytes: int, device: bool = False) -> int:
        return self._submit(True, ptr, device, offset, nbytes)

    def submit_read_strided(self, ptr: int, offset: int, nbytes: int, count: int, stride: int,
                            device: bool = False) -> int:
        """``count`` reads of ``nbytes`` under one ticket: read i fills ``ptr + i * stride`` from file
        offset ``offset + i * stride`` (equally spaced slices of a larger image)."""
        if self._h is None:
            raise ValueError("engine is closed")
        t = lib().daser_io_submit_strided(self._h, 0, C.c_void_p(ptr), int(device), offset, nbytes, count, stride)
        if t < 0:
            raise OSError(-t, os.strerror(-t))
        return t

    def wait(self, ticket: int, timeout_s: Optional[float] = 120.0) -> None:
        ms = -1 if timeout_s is None else int(timeout_s * 1000)
        rc = lib().daser_io_wait(self._h, ticket, ms)
        if rc == 1:
            raise IOTimeout(f"IO ticket {ticket} still pending after {timeout_s}s")
        if rc < 0:
            raise OSError(-rc, os.strerror(-rc), self.path)

    def done(self, ticket: int) -> bool:
        """True once every piece of ``ticket`` has completed (successfully or not); :meth:`wait` still
        has to be called to learn the outcome and release the ticket."""
        rc = lib().daser_io_poll(self._h, ticket)
        if rc < 0:
            raise OSError(-rc, os.strerror(-rc), self.path)
        return rc == 1

    def inject_fault(self, count: int, err_no: int = 0, short_bytes: int = -1) -> None:
        lib().daser_io_inject(self._h, count, err_no, short_bytes)

    def register_buffers(self, regions: Sequence[tuple[int, int]]) -> int:
        """Register host buffers ``(address, bytes)`` with the io_uring ring: IO into them then
        runs as fixed-buffer operations (no page pinning per IO).  Once per engine, before IO into
        them.  Returns the number of registered regions; 0 on other backends or when the kernel
        refuses (memlock limit, too many regions): plain IO keeps working either way."""
        regions = [(p, n) for p, n in regions if p and n > 0]
        if not regions:
            return 0
        ptrs = (C.c_void_p * len(regions))(*[p for p, _ in regions])
        lens = (C.c_int64 * len(regions))(*[n for _, n in regions])
        rc = int(lib().daser_io_register_buffers(self._h, ptrs, lens, len(regions)))
        return max(rc, 0)

    def stats(self) -> dict[str, int]:
        out = (C.c_int64 * 5)()
        lib().daser_io_stats(self._h, out)
        d = dict(zip(("pieces", "bytes_read", "bytes_written", "resubmits", "direct_pieces"), out))
        d["fixed_pieces"] = int(lib().daser_io_fixed_pieces(self._h))
        return d

    def close(self) -> None:
        if self._h is not None:
            lib().daser_io_close(self._h)
            self._h = None

    def __enter__(self) -> "IOEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
