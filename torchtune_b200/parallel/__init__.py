from .dp import DataParallelEngine, FlatParameters, ShardedAdamW
from .fabric import PeerBuffer
from .mesh import ParallelDims
from .strategy import ParallelStrategy, ReplicatedOptimizer, init_from_config

__all__ = ["DataParallelEngine", "FlatParameters", "ShardedAdamW", "PeerBuffer", "ParallelDims", "ParallelStrategy", "ReplicatedOptimizer", "init_from_config"]
