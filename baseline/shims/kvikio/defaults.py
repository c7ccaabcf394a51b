"""``kvikio.defaults``: process-wide settings, same names and default values as kvikio's."""

from __future__ import annotations

import os
import threading
from typing import Any

_lock = threading.Lock()


def _initial() -> dict[str, Any]:
    import kvikio  # the stand-in package itself (CompatMode lives there)

    env = os.environ.get("KVIKIO_COMPAT_MODE", "ON").upper()
    # without an nvidia-fs driver kvikio resolves AUTO to ON; OFF cannot work and is refused at open
    mode = {"OFF": kvikio.CompatMode.OFF, "FALSE": kvikio.CompatMode.OFF, "0": kvikio.CompatMode.OFF,
            "AUTO": kvikio.CompatMode.ON}.get(env, kvikio.CompatMode.ON)
    return {
        "compat_mode": mode,
        "num_threads": int(os.environ.get("KVIKIO_NTHREADS", "1")),
        "task_size": int(os.environ.get("KVIKIO_TASK_SIZE", str(4 << 20))),
        "bounce_buffer_size": int(os.environ.get("KVIKIO_BOUNCE_BUFFER_SIZE", str(16 << 20))),
    }


_values: dict[str, Any] = {}


def _ensure() -> None:
    if not _values:
        _values.update(_initial())


def get(name: str) -> Any:
    with _lock:
        _ensure()
        if name not in _values:
            raise KeyError(name)
        return _values[name]


def set(*args: Any) -> None:  # noqa: A001  (kvikio's own name)
    """``set("name", value)`` or ``set({"name": value, ...})``."""
    with _lock:
        _ensure()
        if len(args) == 1 and isinstance(args[0], dict):
            _values.update(args[0])
        elif len(args) == 2:
            _values[args[0]] = args[1]
        else:
            raise TypeError("set(name, value) or set({name: value})")
        generation[0] += 1


generation = [0]  # bumped by set(); the thread pool is rebuilt when num_threads changed
