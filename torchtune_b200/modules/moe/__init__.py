from .experts import GroupedExperts, LoRAGroupedExperts
from .indices import generate_permute_indices
from .moe import MoE, TokenChoiceTopKRouter
from .utils import expert_load_imbalance, should_use_grouped_mm

__all__ = ["GroupedExperts", "LoRAGroupedExperts", "MoE", "TokenChoiceTopKRouter", "expert_load_imbalance", "generate_permute_indices", "should_use_grouped_mm"]
