"""Stand-in for the part of ``kvikio`` the reference uses, doing what kvikio's compatibility
mode does: POSIX reads and writes on a thread pool through a pinned host bounce buffer.

The reference's transfer layer (``daser/connector/gds_transfer.py:10-13, 52-62, 92, 115``)
needs ``kvikio.defaults.get("compat_mode")``, ``kvikio.defaults.set("num_threads", n)``,
``kvikio.CompatMode`` and ``kvikio.cufile.CuFile(path, "r+")`` with ``pread`` / ``pwrite``
returning a future that has ``get()``.  kvikio cannot be installed offline and the GPU boxes
have no nvidia-fs driver, so compatibility mode is also what the real package would run there.
This package is only ever put on ``sys.path`` by the reference arm of the benchmark; it imports
nothing from the framework under test and loads none of its libraries.
"""

from __future__ import annotations

import enum

from . import defaults  # noqa: F401  (kvikio.defaults)

__version__ = "0.0-shim"


class CompatMode(enum.Enum):
    OFF = 0
    ON = 1
    AUTO = 2


from . import cufile  # noqa: E402,F401  (kvikio.cufile)
