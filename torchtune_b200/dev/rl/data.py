"""Prompt datasets for reinforcement learning under the module path the reference uses (torchtune/dev/rl/data.py:25-113); the code
lives in :mod:`torchtune_b200.dev.grpo.data`."""
from ..grpo.data import ReasoningProblem, RLDataset, padded_collate_rl, reasoning_dataset

__all__ = ["ReasoningProblem", "RLDataset", "padded_collate_rl", "reasoning_dataset"]
