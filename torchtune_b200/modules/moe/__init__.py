from .experts import GroupedExperts, LoRAGroupedExperts
from .indices import generate_permute_indices
from .moe import MoE, TokenChoiceTopKRouter
from .utils import should_use_grouped_mm

__all__ = ["GroupedExperts", "LoRAGroupedExperts", "MoE", "TokenChoiceTopKRouter", "generate_permute_indices", "should_use_grouped_mm"]
