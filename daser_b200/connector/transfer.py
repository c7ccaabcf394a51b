"""Data plane: move bytes between the store file and host or GPU memory.

Capability parity: ``daser/connector/gds_transfer.py:22-127`` — ``TransferBackend``,
``GDSTransferLayer(path, nthreads)`` with ``.backend``, ``await write_async(buf, off, n)``,
``await read_into_async(buf, off, n)``, ``.close()``, context manager, and
``FileNotFoundError`` for a missing store.  The reference delegates to kvikio (cuFile or a
POSIX thread pool with a CPU bounce buffer) and hands it cupy views; here the native engine
(:mod:`daser_b200.io.engine`) takes raw pointers, and three things differ:

* the fallback is a real io_uring path (then POSIX), not only a thread pool;
* GPU buffers on a host backend are staged through a small ring of *persistent pinned
  tiles* with the file IO of tile ``i+1`` overlapping the PCIe copy of tile ``i`` on a
  dedicated copy stream, so memory is O(tile) rather than O(chunk);
* stream ordering is explicit: a write first waits for an event recorded on the stream
  that produced the buffer, and a read returns only after its copies are ordered before
  the consumer stream.  The reference issues cuFile IO from another thread with no
  ordering against the copy kernels (``daser_connector.py:634-672``).

Buffers may be torch tensors (CPU or CUDA), numpy arrays, or ``(ptr, is_device)`` pairs.
"""

from __future__ import annotations

import asyncio
import enum
import os
import threading
from typing import Any, Optional

from daser_b200 import metrics
from daser_b200.io.engine import IOBackend, IOEngine
from daser_b200.logging import init_logger, init_perf_logger

logger = init_logger(__name__)
_perf = init_perf_logger("transfer")


class TransferBackend(enum.Enum):
    GDS = "gds"
    IO_URING = "io_uring"
    POSIX = "posix"
    COMPAT = "posix"  # the reference's name for its non-GDS path


_FROM_ENGINE = {
    IOBackend.GDS: TransferBackend.GDS,
    IOBackend.IO_URING: TransferBackend.IO_URING,
    IOBackend.POSIX: TransferBackend.POSIX,
}
_TO_ENGINE = {"auto": IOBackend.AUTO, "gds": IOBackend.GDS, "io_uring": IOBackend.IO_URING,
              "posix": IOBackend.POSIX}


def _describe(buf: Any) -> tuple[int, bool, Any]:
    """(address, is_device, torch tensor or None) of a buffer argument."""
    if isinstance(buf, tuple):
        return int(buf[0]), bool(buf[1]), None
    if hasattr(buf, "data_ptr"):
        if not buf.is_contiguous():
            raise ValueError("transfer buffers must be contiguous")
        return buf.data_ptr(), bool(buf.is_cuda), buf
    if hasattr(buf, "ctypes"):
        return buf.ctypes.data, False, None
    raise TypeError(f"unsupported buffer type {type(buf)!r}")


class TransferLayer:
    """One open store file with a fixed backend."""

    def __init__(self, path: str, nthreads: int = 4, backend: str = "auto",
                 device: Optional[int] = None, tile_bytes: int = 8 << 20, num_tiles: int = 4,
                 queue_depth: int = 64) -> None:
        if not os.path.exists(path):
            raise FileNotFoundError(f"store file not found: {path}")
        want = _TO_ENGINE[os.environ.get("DASER_IO_BACKEND", backend)]
        self._device = device
        try:
            self._io = IOEngine(path, want, device=device, queue_depth=queue_depth, nthreads=nthreads)
        except OSError:
            if want is not IOBackend.AUTO:
                raise
            self._io = IOEngine(path, IOBackend.POSIX, nthreads=nthreads)
        self._backend = _FROM_ENGINE[self._io.backend]
        self._path = path
        self._tile_bytes = tile_bytes
        self._num_tiles = num_tiles
        self._tiles: list[Any] = []
        self._tile_events: list[Any] = []
        self._copy_stream = None
        self._lock = threading.Lock()
        logger.info("[GDS] store %s opened with backend %s", path, self._backend.name)

    # -- properties ---------------------------------------------------------------------
    @property
    def backend(self) -> TransferBackend:
        return self._backend

    @property
    def engine(self) -> IOEngine:
        return self._io

    # -- pinned staging -------------------------------------------------------------------
    def _ensure_tiles(self):
        import torch

        if not self._tiles:
            self._tiles = [torch.empty(self._tile_bytes, dtype=torch.uint8).pin_memory()
                           for _ in range(self._num_tiles)]
            self._tile_events = [None] * self._num_tiles
            self._copy_stream = torch.cuda.Stream(device=self._device)
        return self._tiles

    # -- synchronous core -------------------------------------------------------------------
    def write(self, buf: Any, file_offset: int, nbytes: int) -> None:
        """Write ``nbytes`` from ``buf`` at ``file_offset``; returns when the data is in the file."""
        ptr, is_dev, tensor = _describe(buf)
        if not is_dev:
            self._io.wait(self._io.submit_write(ptr, file_offset, nbytes))
        elif self._backend is TransferBackend.GDS:
            import torch

            torch.cuda.current_stream().synchronize()  # cuFile is not stream ordered
            self._io.wait(self._io.submit_write(ptr, file_offset, nbytes, device=True))
        else:
            self._staged(tensor, ptr, file_offset, nbytes, write=True)
        metrics.inc("transfer.bytes_written", nbytes)

    def read_into(self, buf: Any, file_offset: int, nbytes: int) -> None:
        """Read ``nbytes`` at ``file_offset`` into ``buf``.

        For GPU buffers the copies are ordered before later work on the caller's current
        stream; the host does not block on the GPU.
        """
        ptr, is_dev, tensor = _describe(buf)
        if not is_dev:
            self._io.wait(self._io.submit_read(ptr, file_offset, nbytes))
        elif self._backend is TransferBackend.GDS:
            import torch

            torch.cuda.current_stream().synchronize()
            self._io.wait(self._io.submit_read(ptr, file_offset, nbytes, device=True))
        else:
            self._staged(tensor, ptr, file_offset, nbytes, write=False)
        metrics.inc("transfer.bytes_read", nbytes)

    def _staged(self, tensor: Any, ptr: int, file_offset: int, nbytes: int, write: bool) -> None:
        """GPU buffer on a host backend: pipeline file IO and PCIe copies through pinned tiles."""
        import torch

        if tensor is None:
            raise TypeError("device buffers on a host backend must be torch tensors")
        flat = tensor.view(torch.uint8).reshape(-1)
        if flat.numel() < nbytes:
            raise ValueError("buffer smaller than the transfer")
        with self._lock:
            tiles = self._ensure_tiles()
            cs = self._copy_stream
            producer = torch.cuda.current_stream()
            ready = torch.cuda.Event()
            ready.record(producer)
            cs.wait_event(ready)  # order after whatever produced / last consumed the buffer
            pending: list[tuple[int, int, int, int]] = []  # (tile, ticket, offset in buf, length)
            nt = len(tiles)

            def retire(entry):
                tile, ticket, off, length = entry
                self._io.wait(ticket)
                if not write:
                    with torch.cuda.stream(cs):
                        flat[off : off + length].copy_(tiles[tile][:length], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(cs)
                    self._tile_events[tile] = ev

            pos, i = 0, 0
            while pos < nbytes:
                length = min(self._tile_bytes, nbytes - pos)
                tile = i % nt
                if len(pending) == nt:
                    retire(pending.pop(0))
                if self._tile_events[tile] is not None:
                    self._tile_events[tile].synchronize()  # the tile's last copy has drained
                    self._tile_events[tile] = None
                if write:
                    with torch.cuda.stream(cs):
                        tiles[tile][:length].copy_(flat[pos : pos + length], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(cs)
                    ev.synchronize()
                    ticket = self._io.submit_write(tiles[tile].data_ptr(), file_offset + pos, length)
                else:
                    ticket = self._io.submit_read(tiles[tile].data_ptr(), file_offset + pos, length)
                pending.append((tile, ticket, pos, length))
                pos += length
                i += 1
            for entry in pending:
                retire(entry)
            if not write:
                done = torch.cuda.Event()
                done.record(cs)
                producer.wait_event(done)

    # -- asyncio API (reference surface) ---------------------------------------------------------
    async def write_async(self, buf: Any, file_offset: int, nbytes: int) -> None:
        loop = asyncio.get_running_loop()
        await loop.run_in_executor(None, self._in_device_ctx, self.write, buf, file_offset, nbytes)

    async def read_into_async(self, buf: Any, file_offset: int, nbytes: int) -> None:
        loop = asyncio.get_running_loop()
        await loop.run_in_executor(None, self._in_device_ctx, self.read_into, buf, file_offset, nbytes)

    def _in_device_ctx(self, fn, buf, file_offset, nbytes):
        if self._device is not None:
            import torch

            with torch.cuda.device(self._device):
                return fn(buf, file_offset, nbytes)
        return fn(buf, file_offset, nbytes)

    # -- lifecycle ------------------------------------------------------------------------------------
    def close(self) -> None:
        if self._io is not None:
            for ev in self._tile_events:
                if ev is not None:
                    ev.synchronize()
            self._io.close()
            self._io = None  # type: ignore[assignment]

    def __enter__(self) -> "TransferLayer":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()


# The reference's class name.
GDSTransferLayer = TransferLayer
