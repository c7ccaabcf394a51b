"""The cuFile (GPUDirect Storage) backend of the native IO engine, against a stand-in library.

The boxes this project runs on have no nvidia-fs driver, so the real ``libcufile`` cannot move a
byte there.  What can be checked anywhere is the engine's side of the contract: it loads the
library by name, opens the driver, registers the file descriptor, routes *device* pieces through
``cuFileRead`` / ``cuFileWrite`` with the right pointer, size and file offset, reports a failing
call as an IO error, and closes everything.  The stand-in implements those six entry points over
``pread`` / ``pwrite`` ("device" pointers are host pointers) and logs each call.  It is found
through ``LD_LIBRARY_PATH``, so the engine runs in a child process.
"""

import os
import shutil
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE = r"""
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/types.h>
#include <unistd.h>
typedef struct { int err; int cu_err; } CUfileError_t;
typedef struct { int type; union { int fd; void* handle; } handle; const void* fs_ops; } CUfileDescr_t;
static int g_open = 0;
static int g_fail_reads = -1;
static void note(const char* what, long a, long b) {
  const char* path = getenv("FAKE_CUFILE_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (f) { fprintf(f, "%s %ld %ld\n", what, a, b); fclose(f); }
}
CUfileError_t cuFileDriverOpen(void) { g_open = 1; note("driver_open", 0, 0); CUfileError_t e = {0, 0}; return e; }
CUfileError_t cuFileDriverClose(void) { g_open = 0; note("driver_close", 0, 0); CUfileError_t e = {0, 0}; return e; }
CUfileError_t cuFileHandleRegister(void** fh, CUfileDescr_t* d) {
  CUfileError_t e = {0, 0};
  if (!g_open || d->type != 1) { e.err = 5001; return e; }
  int* h = (int*)malloc(sizeof(int));
  *h = d->handle.fd;
  *fh = h;
  note("register", d->handle.fd, 0);
  return e;
}
void cuFileHandleDeregister(void* fh) { note("deregister", 0, 0); free(fh); }
ssize_t cuFileRead(void* fh, void* dev, size_t n, off_t file_off, off_t dev_off) {
  if (g_fail_reads < 0) { const char* s = getenv("FAKE_CUFILE_FAIL_READS"); g_fail_reads = s ? atoi(s) : 0; }
  if (g_fail_reads > 0) { --g_fail_reads; errno = EIO; return -1; }
  note("read", (long)n, (long)file_off);
  return pread(*(int*)fh, (char*)dev + dev_off, n, file_off);
}
ssize_t cuFileWrite(void* fh, const void* dev, size_t n, off_t file_off, off_t dev_off) {
  note("write", (long)n, (long)file_off);
  return pwrite(*(int*)fh, (const char*)dev + dev_off, n, file_off);
}
"""

CHILD = """
import ctypes, os, sys
sys.path.insert(0, {root!r})
import numpy as np
from daser_b200.io.engine import IOBackend, IOEngine, preallocate

def aligned(n):
    # the engine hands cuFile its O_DIRECT descriptor; the stand-in's "device" memory is host
    # memory, so it has to satisfy O_DIRECT's alignment itself
    raw = np.zeros(n + 4096, dtype=np.uint8)
    off = (-raw.ctypes.data) % 4096
    return raw[off : off + n]

path = sys.argv[1]
preallocate(path, 8 << 20)
io = IOEngine(path, IOBackend.GDS, device=0)
assert io.backend is IOBackend.GDS, io.backend
src = aligned(5 << 20)   # spans three 2 MiB pieces
src[:] = np.random.default_rng(0).integers(0, 256, 5 << 20, dtype=np.uint8)
io.wait(io.submit_write(src.ctypes.data, 4096, src.size, device=True))
dst = aligned(src.size)
io.wait(io.submit_read(dst.ctypes.data, 4096, dst.size, device=True))
assert np.array_equal(src, dst)
part = aligned(3 * 4096).reshape(3, 4096)
io.wait(io.submit_read_strided(part.ctypes.data, 4096 + 8192, 1024, 3, 4096, device=True))
want = src[8192:8192 + 3 * 4096].reshape(3, 4096)
assert np.array_equal(part[:, :1024], want[:, :1024]) and not part[:, 1024:].any()
if os.environ.get("FAKE_CUFILE_FAIL_READS"):
    try:
        io.wait(io.submit_read(dst.ctypes.data, 0, 4096, device=True))
    except OSError as exc:
        print("READ_FAILED", exc.errno)
st = io.stats()
io.close()
print("GDS_OK", st["bytes_read"], st["bytes_written"])
"""


@pytest.fixture(scope="module")
def fake_cufile(tmp_path_factory):
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    d = tmp_path_factory.mktemp("fakecufile")
    (d / "fake_cufile.c").write_text(FAKE)
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(d / "libcufile.so.0"), str(d / "fake_cufile.c")], check=True)
    return d


def _run(fake_dir, tmp_path, **env):
    log = tmp_path / "calls.log"
    script = tmp_path / "child.py"
    script.write_text(textwrap.dedent(CHILD.format(root=ROOT)))
    e = dict(os.environ, LD_LIBRARY_PATH=f"{fake_dir}:{os.environ.get('LD_LIBRARY_PATH', '')}",
             FAKE_CUFILE_LOG=str(log), **env)
    proc = subprocess.run([sys.executable, str(script), str(tmp_path / "daser.store")], capture_output=True, text=True,
                          timeout=120, env=e)
    calls = [l.split() for l in log.read_text().splitlines()] if log.exists() else []
    return proc, calls


def test_device_pieces_go_through_cufile(fake_cufile, tmp_path):
    proc, calls = _run(fake_cufile, tmp_path)
    assert proc.returncode == 0 and "GDS_OK" in proc.stdout, proc.stdout + proc.stderr
    names = [c[0] for c in calls]
    assert names[0] == "driver_open" and names[1] == "register"
    assert names.count("deregister") == 1 and names[-1] in ("driver_close", "deregister")
    writes = sorted((int(c[2]), int(c[1])) for c in calls if c[0] == "write")
    assert writes == [(4096, 2 << 20), (4096 + (2 << 20), 2 << 20), (4096 + (4 << 20), 1 << 20)]  # offset, size per piece
    reads = [(int(c[2]), int(c[1])) for c in calls if c[0] == "read"]
    assert sorted(reads[:3]) == writes
    assert sorted(reads[3:]) == [(4096 + 8192 + i * 4096, 1024) for i in range(3)]  # the strided extents
    total = proc.stdout.split("GDS_OK")[1].split()
    assert int(total[0]) == (5 << 20) + 3 * 1024 and int(total[1]) == 5 << 20


def test_a_failing_cufile_read_is_an_io_error(fake_cufile, tmp_path):
    """``cuFileRead`` returning -1 with errno set surfaces as ``OSError`` with that errno from ``wait``."""
    proc, _ = _run(fake_cufile, tmp_path, FAKE_CUFILE_FAIL_READS="1")
    assert proc.returncode != 0 and "Input/output error" in proc.stderr, proc.stdout + proc.stderr


def test_gds_is_refused_when_the_library_is_missing(tmp_path):
    from daser_b200.io.engine import IOBackend, IOEngine, preallocate

    p = tmp_path / "s"
    preallocate(str(p), 1 << 20)
    if os.path.exists("/proc/driver/nvidia-fs/stats"):
        pytest.skip("a real GDS driver is present")
    try:
        import ctypes

        ctypes.CDLL("libcufile.so.0")
        pytest.skip("a real libcufile is installed: opening its driver without nvidia-fs can stall")
    except OSError:
        pass
    with pytest.raises(OSError):
        IOEngine(str(p), IOBackend.GDS, device=0)
