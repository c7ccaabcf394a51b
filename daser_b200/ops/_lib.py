"""ctypes loader for ``libdaser_ops.so`` and the parameter blocks shared with the kernels.

The library is built in-tree by :mod:`daser_b200.ops.build`.  Every entry point takes raw
device pointers and a CUDA stream, so the same binary serves torch tensors and callers
that have no torch at all.  If the library is missing the import of any op fails loudly:
there is no PyTorch fallback on the GPU path.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

MAX_RANKS = 8
_LIB_PATH = Path(__file__).resolve().parent / "libdaser_ops.so"
_lib: Optional[C.CDLL] = None

launch_count = 0  # kernels launched through this module (bench.py reports it)


class KVPool(C.Structure):
    """Mirror of ``DaserKVPool`` (``ops/csrc/kv_paged.h``)."""

    _fields_ = [
        ("payload", C.c_void_p * MAX_RANKS),
        ("scales", C.c_void_p * MAX_RANKS),
        ("stride_layer", C.c_int64),
        ("stride_block", C.c_int64),
        ("stride_kv", C.c_int64),
        ("stride_tok", C.c_int64),
        ("stride_head", C.c_int64),
        ("num_blocks", C.c_int32),
        ("n_ranks", C.c_int32),
        ("heads_per_rank", C.c_int32),
        ("pool_is_fp8", C.c_int32),
    ]


class KVJob(C.Structure):
    """Mirror of ``DaserKVJob``."""

    _fields_ = [
        ("slot_ptr", C.c_void_p),
        ("block_id", C.c_void_p),
        ("delta", C.c_void_p),
        ("cos_sin", C.c_void_p),
        ("status", C.c_void_p),
        ("max_pos", C.c_int32),
        ("n_slots", C.c_int32),
        ("num_layers", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("block_tokens", C.c_int32),
        ("image_is_fp8", C.c_int32),
        ("rank", C.c_int32),
        ("layer_begin", C.c_int32),
        ("layer_count", C.c_int32),
        ("lg_heads", C.c_int32),
        ("lg_tokens", C.c_int32),
        ("lg_groups", C.c_int32),
        ("reserved", C.c_int32),
    ]


class Gemm(C.Structure):
    """Mirror of ``DaserGemm`` (``ops/csrc/gemm.cu``)."""

    _fields_ = [
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("lda", C.c_int64),
        ("ldb", C.c_int64),
        ("ldc", C.c_int64),
        ("M", C.c_int32),
        ("N", C.c_int32),
        ("K", C.c_int32),
        ("block_n", C.c_int32),
        ("k_splits", C.c_int32),
        ("epilogue", C.c_int32),
        ("n_owners", C.c_int32),
        ("rows_per_owner", C.c_int32),
        ("dst_row_offset", C.c_int32),
        ("c", C.c_void_p * MAX_RANKS),
        ("arrive", C.c_void_p * MAX_RANKS),
        ("status", C.c_void_p),
        ("gate_flags", C.c_void_p),
        ("gate_target", C.c_uint32),
        ("gate_rows", C.c_int32),
        ("gate_base", C.c_void_p),
        ("work", C.c_void_p),
        ("work_ld", C.c_int64),
        ("tile_counters", C.c_void_p),
        ("bcast", C.c_int32),
        ("rope_positions", C.c_void_p),
        ("rope_slot_mapping", C.c_void_p),
        ("rope_cos_sin", C.c_void_p),
        ("rope_q_out", C.c_void_p),
        ("rope_pool", C.c_void_p),
        ("rope_max_pos", C.c_int32),
        ("rope_hq", C.c_int32),
        ("rope_hkv", C.c_int32),
        ("rope_block_tokens", C.c_int32),
        ("rope_layer", C.c_int32),
        ("rope_rank", C.c_int32),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> C.CDLL:
    """The loaded library; builds nothing, raises if the ``.so`` is absent."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m daser_b200.ops.build` "
                "(there is no fallback for the CUDA path)"
            )
        _lib = C.CDLL(str(_LIB_PATH))
    return _lib


class KernelError(RuntimeError):
    pass


_ERRORS = {-1: "bad argument", -2: "unsupported shape or alignment", -3: "size beyond the supported maximum"}


def check(code: int, what: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code}")


def stream_ptr(stream=None) -> C.c_void_p:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)
