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


def test_registered_buffers_use_fixed_operations(tmp_path):
    """IO into a registered region goes out as READ_FIXED / WRITE_FIXED; IO that leaves the region
    falls back to plain operations; the data is the same either way."""
    import ctypes

    import torch

    path = str(tmp_path / "fixed.store")
    preallocate(path, 16 << 20)
    buf = torch.empty(9 << 20, dtype=torch.uint8)
    base = (buf.data_ptr() + 4095) // 4096 * 4096
    try:
        eng = IOEngine(path, IOBackend.IO_URING)
    except OSError:
        pytest.skip("io_uring unavailable")
    with eng:
        n = eng.register_buffers([(base, 4 << 20)])
        if n == 0:
            pytest.skip("the kernel refused to register buffers (memlock limit)")
        assert n == 1
        assert eng.register_buffers([(base, 4096)]) == 0  # one registration per ring
        src = (ctypes.c_uint8 * (4 << 20)).from_address(base)
        for i in range(0, 4 << 20, 997):
            src[i] = i % 251
        eng.wait(eng.submit_write(base, 0, 4 << 20))           # inside the region: fixed
        fixed_after_write = eng.stats()["fixed_pieces"]
        assert fixed_after_write >= 1
        out = base + (4 << 20)                                  # outside the region: plain
        eng.wait(eng.submit_read(out, 0, 4 << 20))
        assert eng.stats()["fixed_pieces"] == fixed_after_write
        dst = (ctypes.c_uint8 * (4 << 20)).from_address(out)
        assert all(dst[i] == src[i] for i in range(0, 4 << 20, 997))
        eng.wait(eng.submit_read(base + (3 << 20), 1 << 20, 2 << 20))  # crosses the region's end: plain
        assert eng.stats()["fixed_pieces"] == fixed_after_write
        eng.inject_fault(1, 0, 4096)                            # a short fixed read is resubmitted inside the region
        eng.wait(eng.submit_read(base, 0, 1 << 20))
        st = eng.stats()
        assert st["fixed_pieces"] > fixed_after_write and st["resubmits"] >= 1


@pytest.mark.parametrize("backend", _backends())
def test_strided_read_fills_equally_spaced_slices_under_one_ticket(store, backend):
    """Some layers of every slot of a chunk: extent i of the file lands at the same offset of the
    image in memory; everything between the extents stays untouched."""
    slot, layer, n_slots = 40960, 10240, 6
    rng = np.random.default_rng(1)
    data = rng.integers(0, 256, n_slots * slot, dtype=np.uint8)
    with _open(store, backend) as io:
        src = _aligned(n_slots * slot)
        src[:] = data
        io.wait(io.submit_write(src.ctypes.data, 8192, n_slots * slot))
        dst = _aligned(n_slots * slot, fill=0xEE)
        l0, count = 1, 2  # layers 1 and 2 of every slot
        io.wait(io.submit_read_strided(dst.ctypes.data + l0 * layer, 8192 + l0 * layer, count * layer, n_slots, slot))
        got, want = dst.reshape(n_slots, slot), data.reshape(n_slots, slot)
        assert np.array_equal(got[:, l0 * layer : (l0 + count) * layer], want[:, l0 * layer : (l0 + count) * layer])
        assert (got[:, : l0 * layer] == 0xEE).all() and (got[:, (l0 + count) * layer :] == 0xEE).all()
        # an injected error on one extent fails the whole ticket
        io.inject_fault(1, errno.EIO)
        with pytest.raises(OSError):
            io.wait(io.submit_read_strided(dst.ctypes.data, 8192, layer, n_slots, slot))
        with pytest.raises(OSError):
            io.submit_read_strided(dst.ctypes.data, 0, 4096, 2, 1024)  # extents would overlap


@pytest.mark.parametrize("backend", _backends())
def test_done_polls_without_consuming_the_ticket(store, backend):
    import time

    with _open(store, backend) as eng:
        buf = _aligned(1 << 20, fill=7)
        eng.wait(eng.submit_write(buf.ctypes.data, 0, 1 << 20))
        dst = _aligned(1 << 20, fill=0)
        t = eng.submit_read(dst.ctypes.data, 0, 1 << 20)
        deadline = time.time() + 10
        while not eng.done(t):
            assert time.time() < deadline
            time.sleep(0.001)
        assert eng.done(t)      # still there: polling releases nothing
        eng.wait(t)             # the outcome is collected by wait, once
        assert (dst == 7).all()
        with pytest.raises(OSError) as exc:
            eng.done(t)
        assert exc.value.errno == errno.ENOENT
