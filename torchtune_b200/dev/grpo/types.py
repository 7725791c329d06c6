"""Containers of the GRPO loop (parity: torchtune/dev/grpo/types.py:13-60)."""
from typing import Any, List, NamedTuple, Optional

import torch


class GRPOTrajectory(NamedTuple):
    """``B`` prompts × ``G`` sampled completions: sequences ``[B·G, P+L]``, per-token log-probs of the sampling policy and of the
    reference ``[B·G, L]``, group-normalised advantages ``[B·G]``, attention mask / positions, response padding mask, lengths."""

    query_responses: torch.Tensor = None
    logprobs: torch.Tensor = None
    ref_logprobs: torch.Tensor = None
    advantages: torch.Tensor = None
    masks: torch.Tensor = None
    position_ids: torch.Tensor = None
    response_padding_masks: torch.Tensor = None
    seq_lens: torch.Tensor = None
    answers: Optional[List[str]] = None


class GRPOStats(NamedTuple):
    loss: torch.Tensor
    policy_loss: torch.Tensor
    kl_loss: torch.Tensor
    ratios: torch.Tensor
    clipfrac: torch.Tensor
    approx_policy_kls: torch.Tensor
    metadata: Optional[dict] = None
