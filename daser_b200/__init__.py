"""daser_b200 — a Blackwell-native RAG KV-cache service.

Layers (lowest first):

* ``config`` / ``logging`` / ``metrics`` / ``hashing`` — cross-cutting.
* ``io`` — native storage engine (cuFile, io_uring, POSIX) behind one API.
* ``kv`` — slot/chunk byte layout, block-scaled fp8 codec, RoPE, HBM tier.
* ``ops`` — hand-written sm_100a kernels and their Python entry points.
* ``parallel`` — symmetric peer memory and fused compute+collective kernels.
* ``proto`` / ``server`` / ``retrieval`` / ``position`` — the control plane.
* ``connector`` — engine-agnostic connector core and the vLLM adapter.
* ``models`` / ``engine`` — the native serving engine (Llama family, paged KV).
* ``service`` — REST front end.

The capability set, wire protocol and on-disk container follow
7774596/DaseR (``daser/``); file:line citations in docstrings point into
that project.
"""

__version__ = "0.1.0"

from daser_b200.config import DaserConfig  # noqa: F401
