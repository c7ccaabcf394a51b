"""Process-wide counters and latency reservoirs.

The reference exposes only ``prefill_ms`` / ``latency_ms`` in two HTTP replies
(``daser/service/http_api.py:176,268``) and has no hit-rate or IO counters.
This registry backs the ``stats`` RPC, the connector's
``get_kv_connector_stats`` hook and the service's ``/metrics`` route
(Prometheus text format).
"""

from __future__ import annotations

import threading
from collections import defaultdict, deque
from typing import Iterable

_lock = threading.Lock()
_counters: dict[str, float] = defaultdict(float)
_samples: dict[str, deque] = defaultdict(lambda: deque(maxlen=4096))
_gauges: dict[str, float] = {}


def inc(name: str, value: float = 1.0) -> None:
    with _lock:
        _counters[name] += value


def set_gauge(name: str, value: float) -> None:
    """A value that is replaced, not accumulated (ring occupancy, tier fill)."""
    with _lock:
        _gauges[name] = float(value)


def observe(name: str, value: float) -> None:
    with _lock:
        _samples[name].append(value)
        _counters[name + ".count"] += 1
        _counters[name + ".sum"] += value


def percentile(values: Iterable[float], q: float) -> float:
    """Nearest-rank percentile, ``q`` in [0, 100]; 0.0 for an empty input."""
    data = sorted(values)
    if not data:
        return 0.0
    rank = max(0, min(len(data) - 1, int(round(q / 100.0 * (len(data) - 1)))))
    return float(data[rank])


def snapshot() -> dict[str, float]:
    with _lock:
        out = dict(_counters)
        out.update(_gauges)
        for name, dq in _samples.items():
            vals = list(dq)
            out[name + ".p50"] = percentile(vals, 50)
            out[name + ".p99"] = percentile(vals, 99)
    return out


def reset() -> None:
    with _lock:
        _counters.clear()
        _samples.clear()
        _gauges.clear()


def prometheus_text(prefix: str = "daser") -> str:
    lines = []
    for key, val in sorted(snapshot().items()):
        safe = "".join(c if c.isalnum() else "_" for c in key)
        lines.append(f"{prefix}_{safe} {val:.9g}")
    return "\n".join(lines) + "\n"
