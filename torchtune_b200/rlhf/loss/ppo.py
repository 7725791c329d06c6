"""PPO clipped objective (parity: torchtune/rlhf/loss/ppo.py:14-122)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ..rewards import masked_mean


class PPOLoss(nn.Module):
    """``max(-A·r, -A·clip(r, 1±ε))`` for the policy plus ``value_coeff`` times the clipped
    value loss ``½·max((V-R)², (clip(V, V_old±c)-R)²)``; means are taken over unmasked tokens."""

    def __init__(self, epsilon: float = 0.1, value_clip_range: float = 0.2, value_coeff: float = 0.1):
        super().__init__()
        self.epsilon = epsilon
        self.value_clip_range = value_clip_range
        self.value_coeff = value_coeff

    def forward(self, pi_old_logprobs: torch.Tensor, pi_logprobs: torch.Tensor, advantages: torch.Tensor, phi_old_values: torch.Tensor, phi_values: torch.Tensor, returns: torch.Tensor, padding_masks: Optional[torch.Tensor] = None, value_padding_masks: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        def mean(x, mask):
            return x.mean() if mask is None else masked_mean(x, mask)

        ratios = torch.exp(pi_logprobs - pi_old_logprobs)
        unclipped = -advantages * ratios
        clipped = -advantages * torch.clamp(ratios, 1.0 - self.epsilon, 1.0 + self.epsilon)
        clipfrac = mean((clipped > unclipped).to(pi_logprobs.dtype), padding_masks)
        policy_loss = mean(torch.maximum(clipped, unclipped), padding_masks)
        v_clipped = torch.clamp(phi_values, phi_old_values - self.value_clip_range, phi_old_values + self.value_clip_range)
        value_loss = 0.5 * mean(torch.maximum((phi_values - returns) ** 2, (v_clipped - returns) ** 2), value_padding_masks)
        loss = policy_loss + self.value_coeff * value_loss
        return loss, policy_loss.detach(), value_loss.detach(), ratios.mean().detach(), clipfrac.detach()
