from . import loss, utils
from ._types import ChosenRejectedOutputs, PPOStats, Trajectory
from .rewards import estimate_advantages, get_reward_penalty_mask, get_rewards_ppo, masked_mean, masked_sum, masked_var, whiten
from .sequence_processing import (
    batched_logits_to_logprobs,
    get_batch_log_probs,
    logits_to_logprobs,
    truncate_sequence_at_first_stop_token,
    truncate_sequence_for_logprobs,
)

__all__ = [
    "loss",
    "utils",
    "ChosenRejectedOutputs",
    "PPOStats",
    "Trajectory",
    "estimate_advantages",
    "get_reward_penalty_mask",
    "get_rewards_ppo",
    "masked_mean",
    "masked_sum",
    "masked_var",
    "whiten",
    "batched_logits_to_logprobs",
    "get_batch_log_probs",
    "logits_to_logprobs",
    "truncate_sequence_at_first_stop_token",
    "truncate_sequence_for_logprobs",
]
