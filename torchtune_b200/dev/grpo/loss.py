"""Group-relative policy optimisation losses (parity: torchtune/dev/grpo/loss.py:15-430; arXiv 2402.03300).

All variants combine a (clipped) importance-weighted advantage term with the unbiased KL estimator
``k3 = exp(ref - pi) - (ref - pi) - 1`` against the reference policy and return
``(loss, policy_loss, kl_loss, ratios, clipfrac)``:

* :class:`GRPOLoss` — token level: ratio and clipping per token, masked mean over all response tokens;
* :class:`GRPOCompletionLoss` — completion level: log-probs are summed over the completion first;
* :class:`GRPOSimpleLoss` — single on-policy step (``pi_old == pi``): no clipping, per-sequence means.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ...rlhf.rewards import masked_mean, masked_sum

_Out = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


def _k3(ref: torch.Tensor, pi: torch.Tensor) -> torch.Tensor:
    d = ref - pi
    return torch.exp(d) - d - 1


def _mean(x: torch.Tensor, mask: Optional[torch.Tensor], dim: Optional[int] = None) -> torch.Tensor:
    if mask is None:
        return x.mean() if dim is None else x.mean(dim)
    return masked_mean(x, mask, dim)


class _Base(nn.Module):
    def __init__(self, epsilon: float = 0.1, kl_coeff: float = 0.1):
        super().__init__()
        self.epsilon, self.kl_coeff = epsilon, kl_coeff

    def _clipped(self, ratios: torch.Tensor, advantages: torch.Tensor):
        clipped = advantages * torch.clamp(ratios, 1.0 - self.epsilon, 1.0 + self.epsilon)
        unclipped = advantages * ratios
        return torch.minimum(clipped, unclipped), (clipped < unclipped).float()


class GRPOLoss(_Base):
    def forward(self, pi_old_logprobs, pi_logprobs, ref_logprobs, advantages, padding_masks: Optional[torch.Tensor] = None) -> _Out:
        ratios = torch.exp(pi_logprobs - pi_old_logprobs)
        per_token, clipped = self._clipped(ratios, advantages[:, None])
        policy = _mean(per_token, padding_masks)
        kl = _mean(_k3(ref_logprobs, pi_logprobs), padding_masks)
        return -(policy - self.kl_coeff * kl), policy.detach(), kl.detach(), ratios.mean().detach(), _mean(clipped, padding_masks).detach()


class GRPOCompletionLoss(_Base):
    def forward(self, pi_old_logprobs, pi_logprobs, ref_logprobs, advantages, padding_masks: Optional[torch.Tensor] = None) -> _Out:
        ones = torch.ones_like(pi_logprobs, dtype=torch.bool) if padding_masks is None else padding_masks
        old, new, ref = (masked_sum(t, ones, dim=1) for t in (pi_old_logprobs, pi_logprobs, ref_logprobs))
        ratios = torch.exp(new - old)
        per_seq, clipped = self._clipped(ratios, advantages)
        policy = per_seq.mean()
        kl = _k3(ref, new).mean()
        return -(policy - self.kl_coeff * kl), policy.detach(), kl.detach(), ratios.mean().detach(), clipped.mean().detach()


class GRPOSimpleLoss(_Base):
    def forward(self, pi_old_logprobs, pi_logprobs, ref_logprobs, advantages, padding_masks: Optional[torch.Tensor] = None) -> _Out:
        kl_tok = _k3(ref_logprobs.detach(), pi_logprobs)
        policy_tok = torch.exp(pi_logprobs - pi_logprobs.detach()) * advantages[:, None]
        loss = _mean(-(policy_tok - self.kl_coeff * kl_tok), padding_masks, dim=1).mean()
        policy = _mean(policy_tok, padding_masks, dim=1).mean().detach()
        kl = _mean(kl_tok, padding_masks, dim=1).mean().detach()
        return loss, policy, kl, torch.tensor(1.0), torch.tensor(0.0)
