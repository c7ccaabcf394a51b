"""``kvikio.cufile.CuFile`` in compatibility mode.

A transfer of ``size`` bytes is cut into tasks of ``defaults.get("task_size")`` bytes (4 MiB)
that run on a pool of ``defaults.get("num_threads")`` threads.  A task on a device buffer goes
through a pinned host bounce buffer: ``pread`` into it, then a host-to-device copy on the
thread's own stream, then a stream synchronise (reads); the mirror image for writes.  A task on
a host buffer is a plain ``pread`` / ``pwrite``.  Buffers are anything that publishes
``__cuda_array_interface__`` or the Python buffer protocol.
"""

from __future__ import annotations

import os
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Optional

from . import defaults

_pool_lock = threading.Lock()
_pool: Optional[ThreadPoolExecutor] = None
_pool_threads = 0
_tls = threading.local()


def _executor() -> ThreadPoolExecutor:
    global _pool, _pool_threads
    n = max(1, int(defaults.get("num_threads")))
    with _pool_lock:
        if _pool is None or _pool_threads != n:
            if _pool is not None:
                _pool.shutdown(wait=True)
            _pool = ThreadPoolExecutor(max_workers=n, thread_name_prefix="kvikio-compat")
            _pool_threads = n
        return _pool


class IOFuture:
    """Completion of one ``pread`` / ``pwrite``: ``get()`` returns the byte count."""

    def __init__(self, parts: list[Future]) -> None:
        self._parts = parts

    def get(self) -> int:
        return sum(p.result() for p in self._parts)

    def done(self) -> bool:
        return all(p.done() for p in self._parts)


def _describe(buf: Any) -> tuple[str, Any, int]:
    """('cuda', torch uint8 view, nbytes) or ('host', memoryview, nbytes)."""
    if hasattr(buf, "__cuda_array_interface__"):
        import torch

        t = torch.as_tensor(buf, device="cuda") if not isinstance(buf, torch.Tensor) else buf
        t = t.reshape(-1).view(torch.uint8)
        return "cuda", t, t.numel()
    mv = memoryview(buf).cast("B")
    return "host", mv, mv.nbytes


def _bounce(nbytes: int):
    """This thread's pinned bounce buffer and copy stream."""
    import torch

    size = max(int(defaults.get("task_size")), nbytes)
    if getattr(_tls, "buf", None) is None or _tls.buf.numel() < size:
        _tls.buf = torch.empty(size, dtype=torch.uint8).pin_memory()
    return _tls.buf


def _stream(device):
    import torch

    key = f"stream{device.index}"
    if getattr(_tls, key, None) is None:
        setattr(_tls, key, torch.cuda.Stream(device=device))
    return getattr(_tls, key)


class CuFile:
    def __init__(self, path: str, flags: str = "r") -> None:
        import kvikio

        if defaults.get("compat_mode") == kvikio.CompatMode.OFF:
            raise RuntimeError("kvikio stand-in: GDS mode needs the real kvikio and an nvidia-fs driver")
        mode = {"r": os.O_RDONLY, "r+": os.O_RDWR, "w": os.O_WRONLY | os.O_CREAT | os.O_TRUNC,
                "w+": os.O_RDWR | os.O_CREAT | os.O_TRUNC, "a": os.O_WRONLY | os.O_CREAT | os.O_APPEND}[flags]
        self._fd = os.open(path, mode, 0o644)
        self._closed = False

    # -- tasks -----------------------------------------------------------------------------
    def _read_task(self, kind: str, view: Any, buf_off: int, nbytes: int, file_off: int) -> int:
        if kind == "host":
            return os.preadv(self._fd, [view[buf_off : buf_off + nbytes]], file_off)
        import torch

        host = _bounce(nbytes)
        done = 0
        mv = memoryview(host.numpy())
        while done < nbytes:
            got = os.preadv(self._fd, [mv[done:nbytes]], file_off + done)
            if got <= 0:
                break
            done += got
        stream = _stream(view.device)
        with torch.cuda.stream(stream):
            view[buf_off : buf_off + done].copy_(host[:done], non_blocking=True)
        stream.synchronize()
        return done

    def _write_task(self, kind: str, view: Any, buf_off: int, nbytes: int, file_off: int) -> int:
        if kind == "host":
            return os.pwritev(self._fd, [view[buf_off : buf_off + nbytes]], file_off)
        import torch

        host = _bounce(nbytes)
        stream = _stream(view.device)
        with torch.cuda.stream(stream):
            host[:nbytes].copy_(view[buf_off : buf_off + nbytes], non_blocking=True)
        stream.synchronize()
        mv = memoryview(host.numpy())
        done = 0
        while done < nbytes:
            put = os.pwritev(self._fd, [mv[done:nbytes]], file_off + done)
            if put <= 0:
                break
            done += put
        return done

    def _submit(self, task, buf: Any, size: Optional[int], file_offset: int, dev_offset: int) -> IOFuture:
        if self._closed:
            raise RuntimeError("file is closed")
        kind, view, total = _describe(buf)
        if kind == "cuda":
            import torch

            # legacy-default-stream semantics of cudaMemcpy in kvikio: work queued before the call is seen
            torch.cuda.current_stream(view.device).synchronize()
        nbytes = total - dev_offset if size is None else int(size)
        task_size = max(4096, int(defaults.get("task_size")))
        ex = _executor()
        parts = []
        for off in range(0, nbytes, task_size):
            n = min(task_size, nbytes - off)
            parts.append(ex.submit(task, kind, view, dev_offset + off, n, file_offset + off))
        return IOFuture(parts)

    # -- kvikio's surface --------------------------------------------------------------------
    def pread(self, buf: Any, size: Optional[int] = None, file_offset: int = 0, task_size: Optional[int] = None,
              dev_offset: int = 0) -> IOFuture:
        return self._submit(self._read_task, buf, size, file_offset, dev_offset)

    def pwrite(self, buf: Any, size: Optional[int] = None, file_offset: int = 0, task_size: Optional[int] = None,
               dev_offset: int = 0) -> IOFuture:
        return self._submit(self._write_task, buf, size, file_offset, dev_offset)

    def read(self, buf: Any, size: Optional[int] = None, file_offset: int = 0, **_: Any) -> int:
        return self.pread(buf, size, file_offset).get()

    def write(self, buf: Any, size: Optional[int] = None, file_offset: int = 0, **_: Any) -> int:
        return self.pwrite(buf, size, file_offset).get()

    def closed(self) -> bool:
        return self._closed

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            os.close(self._fd)

    def __enter__(self) -> "CuFile":
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()
