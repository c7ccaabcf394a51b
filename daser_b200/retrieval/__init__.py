from daser_b200.retrieval.base import RetrievalIndex  # noqa: F401
from daser_b200.retrieval.chunk_index import ChunkHit, ChunkOffsetIndex  # noqa: F401
from daser_b200.retrieval.prefix import PrefixHashIndex  # noqa: F401
