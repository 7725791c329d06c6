"""Containers exchanged between the RLHF recipes and losses (parity: torchtune/rlhf/_types.py:13-90)."""
from dataclasses import dataclass
from typing import NamedTuple

import torch


class Trajectory(NamedTuple):
    """One batch of rollouts: ``query_responses`` ``[b, ctx+resp]``, per-token ``logprobs`` /
    ``ref_logprobs`` / ``values`` ``[b, resp]``, attention ``masks`` and ``position_ids`` for the
    concatenated sequences, padding masks, the index of the last valid value, reward-model
    ``scores`` ``[b]`` and response lengths."""

    query_responses: torch.Tensor
    logprobs: torch.Tensor
    ref_logprobs: torch.Tensor
    values: torch.Tensor
    masks: torch.Tensor
    position_ids: torch.Tensor
    response_padding_masks: torch.Tensor
    value_padding_masks: torch.Tensor
    value_seq_idxs: torch.Tensor
    scores: torch.Tensor
    seq_lens: torch.Tensor


class PPOStats(NamedTuple):
    loss: torch.Tensor
    policy_loss: torch.Tensor
    value_loss: torch.Tensor
    ratios: torch.Tensor
    clipfrac: torch.Tensor
    approx_policy_kls: torch.Tensor


@dataclass
class ChosenRejectedOutputs:
    """Sequence log-probabilities (``[b]``) and logits of the chosen / rejected halves of a
    concatenated forward pass; the logits may be ``None`` when the fused log-prob path is used."""

    chosen_logps: torch.Tensor
    rejected_logps: torch.Tensor
    chosen_logits: torch.Tensor = None
    rejected_logits: torch.Tensor = None
