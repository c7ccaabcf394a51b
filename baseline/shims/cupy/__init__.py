"""Stand-in for the one ``cupy`` call the reference connector makes.

The reference hands torch memory to kvikio through ``cupy.asarray(tensor)``
(``daser/connector/daser_connector.py:506`` and ``:651``) and otherwise uses ``cupy.ndarray``
only in annotations.  cupy cannot be installed offline, so the reference arm of the benchmark
puts this directory on ``sys.path``.  It imports nothing from the framework under test.

``asarray`` returns a zero-copy view object: it keeps the producer alive and republishes its
``__cuda_array_interface__`` (or the host buffer), which is all a consumer such as the kvikio
stand-in needs.
"""

from __future__ import annotations

from typing import Any

__version__ = "0.0-shim"


class ndarray:
    """Zero-copy view over a device (or host) buffer owned by ``base``."""

    def __init__(self, base: Any) -> None:
        self.base = base
        iface = getattr(base, "__cuda_array_interface__", None)
        if iface is None:
            raise TypeError("cupy stand-in: asarray() needs an object with __cuda_array_interface__")
        self.__cuda_array_interface__ = dict(iface)
        n = 1
        for d in iface["shape"]:
            n *= int(d)
        self.size = n
        self.itemsize = int(iface["typestr"][2:])
        self.nbytes = n * self.itemsize
        self.shape = tuple(iface["shape"])

    def __len__(self) -> int:
        return self.shape[0] if self.shape else 0


def asarray(obj: Any, dtype: Any = None) -> ndarray:
    if isinstance(obj, ndarray):
        return obj
    return ndarray(obj)
