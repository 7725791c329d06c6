from .dp import DataParallelEngine, FlatParameters, ShardedAdamW
from .fabric import PeerBuffer
from .mesh import ParallelDims

__all__ = ["DataParallelEngine", "FlatParameters", "ShardedAdamW", "PeerBuffer", "ParallelDims"]
