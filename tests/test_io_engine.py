"""Native storage engine on host memory: every backend that opens here, plus injected faults."""

import errno
import os

import numpy as np
import pytest

from daser_b200.io.engine import IOBackend, IOEngine, IOTimeout, preallocate


def _aligned(n, fill=None):
    raw = np.empty(n + 4096, dtype=np.uint8)
    off = (-raw.ctypes.data) % 4096
    buf = raw[off : off + n]
    if fill is not None:
        buf[:] = fill
    return buf


def _backends():
    return [IOBackend.IO_URING, IOBackend.POSIX]


def _open(path, backend):
    try:
        return IOEngine(str(path), backend)
    except OSError as exc:
        if backend is IOBackend.IO_URING:
            pytest.skip(f"io_uring not permitted here: {exc}")
        raise


@pytest.fixture
def store(tmp_path):
    p = tmp_path / "daser.store"
    preallocate(str(p), 16 << 20)
    assert os.path.getsize(p) == 16 << 20
    return p


def test_missing_file_raises(tmp_path):
    with pytest.raises(FileNotFoundError):
        IOEngine(str(tmp_path / "nope"))


def test_auto_picks_a_host_backend(store):
    with IOEngine(str(store)) as io:
        assert io.backend in (IOBackend.IO_URING, IOBackend.POSIX)
        assert io.file_size == 16 << 20


@pytest.mark.parametrize("backend", _backends())
def test_roundtrip_many_offsets(store, backend):
    rng = np.random.default_rng(0)
    with _open(store, backend) as io:
        assert io.backend is backend
        cases = [(0, 4096), (4096 * 3, 1 << 20), (5 << 20, (5 << 20) + 4096), (123, 777), (8 << 20, 3_276_800)]
        tickets = []
        for off, n in cases:
            src = _aligned(n)
            src[:] = rng.integers(0, 256, n, dtype=np.uint8)
            tickets.append((off, n, src, io.submit_write(src.ctypes.data, off, n)))
        for _, _, _, t in tickets:
            io.wait(t)
        for off, n, src, _ in tickets[::-1]:
            dst = _aligned(n, 0)
            io.wait(io.submit_read(dst.ctypes.data, off, n))
            if off == 123:  # overlapped by nothing else
                assert np.array_equal(dst, src)
        # last writer wins on the overlapping ranges: re-check a disjoint one precisely
        dst = _aligned(3_276_800, 0)
        io.wait(io.submit_read(dst.ctypes.data, 8 << 20, 3_276_800))
        assert np.array_equal(dst, tickets[-1][2])
        st = io.stats()
        assert st["bytes_written"] >= sum(n for _, n in cases)
        assert st["pieces"] >= len(cases) * 2


@pytest.mark.parametrize("backend", _backends())
def test_injected_eio_is_reported(store, backend):
    with _open(store, backend) as io:
        buf = _aligned(1 << 20, 7)
        io.inject_fault(1, errno.EIO)
        with pytest.raises(OSError) as ei:
            io.wait(io.submit_read(buf.ctypes.data, 0, 1 << 20))
        assert ei.value.errno == errno.EIO
        io.wait(io.submit_read(buf.ctypes.data, 0, 1 << 20))  # engine still usable


@pytest.mark.parametrize("backend", _backends())
def test_short_io_is_resubmitted(store, backend):
    with _open(store, backend) as io:
        src = _aligned(1 << 20)
        src[:] = np.arange(1 << 20, dtype=np.uint32).view(np.uint8)[: 1 << 20]
        io.wait(io.submit_write(src.ctypes.data, 1 << 20, 1 << 20))
        dst = _aligned(1 << 20, 0)
        io.inject_fault(1, 0, short_bytes=1000)  # first completion returns 1000 bytes only
        io.wait(io.submit_read(dst.ctypes.data, 1 << 20, 1 << 20))
        assert np.array_equal(dst, src)
        assert io.stats()["resubmits"] >= 1


@pytest.mark.parametrize("backend", _backends())
def test_read_past_end_fails(store, backend):
    with _open(store, backend) as io:
        buf = _aligned(8192, 0)
        with pytest.raises(OSError):
            io.wait(io.submit_read(buf.ctypes.data, (16 << 20) - 4096, 8192))


def test_wait_unknown_ticket_and_timeout_type(store):
    with IOEngine(str(store), IOBackend.POSIX) as io:
        with pytest.raises(OSError):
            io.wait(12345)
    assert issubclass(IOTimeout, TimeoutError)


def test_device_buffers_rejected_on_host_backends(store):
    with IOEngine(str(store), IOBackend.POSIX) as io:
        buf = _aligned(4096, 0)
        with pytest.raises(OSError) as ei:
            io.submit_read(buf.ctypes.data, 0, 4096, device=True)
        assert ei.value.errno == errno.ENOTSUP
