from .data import ReasoningProblem, RLDataset, gsm8k_dataset, gsm8k_sft, padded_collate_rl, reasoning_dataset
from .loss import GRPOCompletionLoss, GRPOLoss, GRPOSimpleLoss, GRPOWithChunkedOutputLoss
from .rewards import batch_shaped_correctness_reward, extract_tags, shaped_correctness_reward
from .types import GRPOStats, GRPOTrajectory

__all__ = ["GRPOCompletionLoss", "GRPOLoss", "GRPOSimpleLoss", "GRPOWithChunkedOutputLoss", "GRPOStats", "GRPOTrajectory", "ReasoningProblem", "RLDataset", "batch_shaped_correctness_reward", "extract_tags", "gsm8k_dataset", "gsm8k_sft", "padded_collate_rl", "reasoning_dataset", "shaped_correctness_reward"]
