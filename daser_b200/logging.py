"""Logging and lightweight performance records.

Capability parity: ``daser/logging.py:9-78`` (``init_logger``, ``PerfLogger``,
``init_perf_logger``; env ``DASER_LOG_LEVEL`` / ``DASER_PERF_LOG``).  In the
reference ``PerfLogger.record`` is never called; here every record also feeds
the process-wide :mod:`daser_b200.metrics` registry, so the numbers surface
through ``/metrics`` and the connector's stats hook even when the text log is
off.
"""

from __future__ import annotations

import logging
import os
import sys
from typing import Optional

from daser_b200 import metrics

_FORMAT = "%(asctime)s %(levelname)s %(name)s %(message)s"


def init_logger(name: str, level: Optional[str] = None) -> logging.Logger:
    """Return a logger with one stream handler.

    Level resolution: explicit argument, else ``DASER_LOG_LEVEL``, else INFO.
    Calling twice with the same name does not duplicate handlers.
    """
    logger = logging.getLogger(name)
    chosen = (level or os.environ.get("DASER_LOG_LEVEL") or "INFO").upper()
    logger.setLevel(getattr(logging, chosen, logging.INFO))
    if not any(getattr(h, "_daser", False) for h in logger.handlers):
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(logging.Formatter(_FORMAT))
        handler._daser = True  # type: ignore[attr-defined]
        logger.addHandler(handler)
        logger.propagate = False
    return logger


class PerfLogger:
    """Structured performance records, text output gated by ``DASER_PERF_LOG=1``."""

    def __init__(self, name: str) -> None:
        self._name = name
        self._logger = init_logger(f"{name}.perf")
        self.enabled = os.environ.get("DASER_PERF_LOG", "0") == "1"

    def record(self, metric: str, value: float, unit: str = "") -> None:
        metrics.observe(f"{self._name}.{metric}", float(value))
        if self.enabled:
            self._logger.info("[PERF] %s=%.6g%s", metric, value, unit)


def init_perf_logger(name: str) -> PerfLogger:
    return PerfLogger(name)
