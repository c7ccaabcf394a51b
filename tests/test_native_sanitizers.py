"""The C++ storage engine under AddressSanitizer + UBSan and under ThreadSanitizer.

The reference has no race or memory checking of any kind; its IO is a third-party library.
compute-sanitizer is not available for the CUDA side here, so the host runtime is where
sanitizers run: the engine's exerciser (concurrent submitters, short IO, injected errors,
shutdown with work in flight) must come out clean.
"""

import os
import subprocess

import pytest

from daser_b200.ops.build import build_index_selftest, build_io_selftest


@pytest.mark.parametrize("san", ["address,undefined", "thread"])
def test_io_engine_selftest_is_clean(tmp_path, san):
    try:
        exe = build_io_selftest(san)
    except RuntimeError as exc:
        pytest.skip(f"sanitizer build unavailable: {str(exc)[-200:]}")
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    proc = subprocess.run([str(exe), str(tmp_path / "san.store")], capture_output=True, text=True, timeout=120, env=env)
    out = proc.stdout + proc.stderr
    if "unexpected memory mapping" in out or "ThreadSanitizer: unsupported" in out:
        pytest.skip("this kernel's address-space layout is not supported by the sanitizer runtime")
    assert proc.returncode == 0, out[-3000:]
    assert "SELFTEST_OK" in proc.stdout
    assert "ERROR: AddressSanitizer" not in out and "WARNING: ThreadSanitizer" not in out and "runtime error" not in out


@pytest.mark.parametrize("san", ["address,undefined", "thread"])
def test_token_index_selftest_is_clean(san):
    try:
        exe = build_index_selftest(san)
    except RuntimeError as exc:
        pytest.skip(f"sanitizer build unavailable: {str(exc)[-200:]}")
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, env=env)
    out = proc.stdout + proc.stderr
    if "unexpected memory mapping" in out or "ThreadSanitizer: unsupported" in out:
        pytest.skip("this kernel's address-space layout is not supported by the sanitizer runtime")
    assert proc.returncode == 0, out[-3000:]
    assert "SELFTEST_OK" in proc.stdout
    assert "ERROR: AddressSanitizer" not in out and "WARNING: ThreadSanitizer" not in out and "runtime error" not in out
