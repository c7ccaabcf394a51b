"""Host-side tracing: Chrome-trace JSON spans, mirrored as NVTX ranges when CUDA is present.

The reference has no tracing; its optimisation notes were produced by reading the code.
Here every connector hook, RPC, IO batch and engine step is wrapped in :func:`span`.  Tracing
is off unless ``DASER_TRACE=/path/to/trace.json`` is set (or :func:`enable` is called); the file
is written at exit (or by :func:`dump`) and loads in ``chrome://tracing`` / Perfetto.  With
``DASER_NVTX=1`` the same spans are pushed as NVTX ranges so they line up with kernels in a
GPU timeline.
"""

from __future__ import annotations

import atexit
import json
import os
import threading
import time
from contextlib import contextmanager
from typing import Any, Iterator, Optional

_lock = threading.Lock()
_events: list[dict[str, Any]] = []
_path: Optional[str] = os.environ.get("DASER_TRACE") or None
_nvtx = os.environ.get("DASER_NVTX", "0") == "1"
_MAX_EVENTS = 1_000_000


def enabled() -> bool:
    return _path is not None or _nvtx


def enable(path: Optional[str] = None, nvtx: bool = False) -> None:
    global _path, _nvtx
    _path, _nvtx = path, nvtx or _nvtx


def disable() -> None:
    global _path, _nvtx
    _path, _nvtx = None, False


@contextmanager
def span(name: str, category: str = "daser", **args: Any) -> Iterator[None]:
    """Record ``name`` for the duration of the block (no-op when tracing is off)."""
    if _path is None and not _nvtx:
        yield
        return
    pushed = False
    if _nvtx:
        try:
            import torch

            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:
            pushed = False
    t0 = time.perf_counter_ns()
    try:
        yield
    finally:
        t1 = time.perf_counter_ns()
        if pushed:
            import torch

            torch.cuda.nvtx.range_pop()
        if _path is not None:
            with _lock:
                if len(_events) < _MAX_EVENTS:
                    _events.append({"name": name, "cat": category, "ph": "X", "ts": t0 / 1e3,
                                    "dur": (t1 - t0) / 1e3, "pid": os.getpid(),
                                    "tid": threading.get_ident() % 100000, "args": args})


def instant(name: str, **args: Any) -> None:
    if _path is None:
        return
    with _lock:
        _events.append({"name": name, "cat": "daser", "ph": "i", "s": "t", "ts": time.perf_counter_ns() / 1e3,
                        "pid": os.getpid(), "tid": threading.get_ident() % 100000, "args": args})


def dump(path: Optional[str] = None) -> Optional[str]:
    """Write the collected events; returns the path written (None when there is nowhere to write)."""
    target = path or _path
    if target is None:
        return None
    with _lock:
        data = {"traceEvents": list(_events), "displayTimeUnit": "ms"}
    tmp = f"{target}.tmp.{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump(data, f)
    os.replace(tmp, target)
    return target


def clear() -> None:
    with _lock:
        _events.clear()


atexit.register(lambda: dump() if _path is not None and _events else None)
