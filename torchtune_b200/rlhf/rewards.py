"""Reward shaping and advantage estimation for PPO (parity: torchtune/rlhf/rewards.py:12-238)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def get_reward_penalty_mask(padding_masks: torch.Tensor, seq_lens: torch.Tensor, penalise_no_eos: bool = True, min_response_length: Optional[int] = None) -> torch.Tensor:
    """True where a sequence's score should be replaced by the penalty: no EOS was produced
    (the padding mask has no padded position) or the response is shorter than the minimum."""
    penalise = torch.zeros_like(seq_lens, dtype=torch.bool)
    if penalise_no_eos:
        penalise = ~padding_masks.any(-1)
    if min_response_length is not None:
        penalise = penalise | (seq_lens < min_response_length)
    return penalise


def get_rewards_ppo(scores: torch.Tensor, logprobs: torch.Tensor, ref_logprobs: torch.Tensor, kl_coeff: float, valid_score_idxs: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-token reward ``-kl_coeff·(logp - ref_logp)`` with the sequence score added at the last
    valid token (``valid_score_idxs``) or at the final position.  Returns ``(total, kl, kl_reward)``."""
    kl = logprobs - ref_logprobs
    kl_reward = -kl_coeff * kl
    total = kl_reward.clone()
    if valid_score_idxs is not None:
        total.scatter_add_(1, valid_score_idxs.unsqueeze(-1), scores.unsqueeze(-1))
    else:
        total[:, -1] += scores
    return total, kl, kl_reward


def masked_sum(x: torch.Tensor, mask: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return (x * mask).sum(dim=dim) if dim is not None else (x * mask).sum()


def masked_mean(x: torch.Tensor, mask: torch.Tensor, dim: Optional[int] = None) -> torch.Tensor:
    return masked_sum(x, mask, dim) / (mask.sum(dim=dim) + 1e-8 if dim is not None else mask.sum() + 1e-8)


def masked_var(centered: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    """Variance of already mean-centred values over the masked positions."""
    var = masked_mean(centered.pow(2), mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("Cannot compute unbiased variance with zero elements in mask.")
        var = var * (n / (n - 1))
    return var


def whiten(x: torch.Tensor, mask: Optional[torch.Tensor] = None, shift_mean: bool = True) -> torch.Tensor:
    """Normalise to unit variance, optionally over a mask.  Same signature and meaning as the reference
    (torchtune/rlhf/rewards.py:157-179): the mean is removed for the scaling and *added back* when ``shift_mean`` is
    true, so ``shift_mean=False`` gives zero-mean values."""
    if mask is not None:
        mean = masked_mean(x, mask)
        var = masked_var(x - mean, mask) if mask.any() else x.var()
    else:
        mean, var = x.mean(), x.var()
    out = (x - mean) * torch.rsqrt(var + 1e-8)
    return out + mean if shift_mean else out


def estimate_advantages(values: torch.Tensor, rewards: torch.Tensor, gamma: float, lmbda: float, masks: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generalised advantage estimation (arXiv 1506.02438).  Returns whitened advantages (zeroed
    outside ``masks``) and the un-normalised returns ``advantages + values``."""
    steps = values.shape[-1]
    adv = torch.zeros_like(values)
    running = torch.zeros_like(values[:, 0])
    for t in range(steps - 1, -1, -1):
        nxt = values[:, t + 1] if t < steps - 1 else 0.0
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        running = delta + gamma * lmbda * running
        adv[:, t] = running
    returns = adv + values
    adv = whiten(adv, mask=masks)
    if masks is not None:
        adv = adv.masked_fill(~masks, 0.0)
    return adv, returns
