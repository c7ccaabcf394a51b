"""Build the native libraries in-tree with nvcc / g++ for sm_100a.

``python -m daser_b200.ops.build`` compiles every ``.cu`` under ``ops/csrc`` into
``ops/libdaser_ops.so`` and the C++ storage engine under ``io/csrc`` into
``io/libdaser_io.so``.  Objects are rebuilt only when a source or header is newer.
The reference is pure Python and has no build step.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
OPS_SRC = PKG / "ops" / "csrc"
IO_SRC = PKG / "io" / "csrc"
OPS_LIB = PKG / "ops" / "libdaser_ops.so"
IO_LIB = PKG / "io" / "libdaser_io.so"
INDEX_SRC = PKG / "server" / "csrc"
INDEX_LIB = PKG / "server" / "libdaser_index.so"
BUILD_DIR = PKG.parent / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build daser_b200")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build_ops(verbose: bool = False, force: bool = False) -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    headers = sorted(OPS_SRC.glob("*.cuh")) + sorted(OPS_SRC.glob("*.h"))
    sources = sorted(OPS_SRC.glob("*.cu"))
    objs = [BUILD_DIR / (s.stem + ".o") for s in sources]

    def compile_one(pair):
        src, obj = pair
        if force or _stale(obj, [src, *headers]):
            flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
            _run([_nvcc(), *flags, "-I", str(OPS_SRC), "-c", str(src), "-o", str(obj)])
            return True
        return False

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as pool:
        rebuilt = list(pool.map(compile_one, zip(sources, objs)))
    if force or any(rebuilt) or _stale(OPS_LIB, objs):
        _run([_nvcc(), "-shared", "-o", str(OPS_LIB), *map(str, objs), "-lcudart"])
    return OPS_LIB


def build_io(force: bool = False) -> Path:
    sources = sorted(p for p in IO_SRC.glob("*.cc") if not p.name.endswith("_selftest.cc"))
    headers = sorted(IO_SRC.glob("*.h"))
    if not sources:
        return IO_LIB
    if force or _stale(IO_LIB, sources + headers):
        cuda_inc = "/usr/local/cuda/include"
        cmd = [
            "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread",
            "-I", str(IO_SRC),
        ]
        if os.path.isdir(cuda_inc):
            cmd += ["-I", cuda_inc, "-DDASER_HAVE_CUDA_HEADERS=1"]
        cmd += ["-o", str(IO_LIB), *map(str, sources), "-ldl"]
        _run(cmd)
    return IO_LIB


def build_io_selftest(sanitize: str = "address,undefined") -> Path:
    """The storage engine's stand-alone exerciser, instrumented with ``-fsanitize=<sanitize>``."""
    BUILD_DIR.mkdir(exist_ok=True)
    out = BUILD_DIR / f"io_selftest_{sanitize.replace(',', '_')}"
    srcs = [IO_SRC / "io_engine.cc", IO_SRC / "io_engine_selftest.cc"]
    if _stale(out, srcs + sorted(IO_SRC.glob("*.h"))):
        _run(["g++", "-O1", "-g", "-std=c++17", f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-pthread",
              "-I", str(IO_SRC), "-o", str(out), *map(str, srcs), "-ldl"])
    return out


def build_index(force: bool = False) -> Path:
    """The control plane's native parts: the token index (hashing through the system's libxxhash)
    and the lookup-by-key server thread."""
    srcs = [INDEX_SRC / "token_index.cc", INDEX_SRC / "fast_lookup.cc"]
    if force or _stale(INDEX_LIB, srcs):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread",
              "-o", str(INDEX_LIB), *map(str, srcs), "-ldl"])
    return INDEX_LIB


def build_index_selftest(sanitize: str = "address,undefined") -> Path:
    """The token index's stand-alone exerciser, instrumented with ``-fsanitize=<sanitize>``."""
    BUILD_DIR.mkdir(exist_ok=True)
    out = BUILD_DIR / f"index_selftest_{sanitize.replace(',', '_')}"
    srcs = [INDEX_SRC / "token_index.cc", INDEX_SRC / "fast_lookup.cc", INDEX_SRC / "token_index_selftest.cc"]
    if _stale(out, srcs):
        _run(["g++", "-O1", "-g", "-std=c++17", f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-pthread",
              "-o", str(out), *map(str, srcs), "-ldl"])
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_io(force=force)
    build_index(force=force)
    build_ops(verbose=verbose, force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(OPS_LIB, IO_LIB, INDEX_LIB)
