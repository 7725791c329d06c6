from .nf4 import NF4Weight, ShardedNF4Weight, linear_nf4
from .nf4_linear import FrozenNF4Linear

__all__ = ["FrozenNF4Linear", "NF4Weight", "ShardedNF4Weight", "linear_nf4"]
