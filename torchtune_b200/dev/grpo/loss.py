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


class GRPOWithChunkedOutputLoss(nn.Module):
    """GRPO objective evaluated directly on (chunks of) the policy's logits, so the ``[B·G, L, vocab]`` fp32 log-softmax of a
    whole response never exists at once (parity: torchtune/dev/grpo/loss.py:270-430).

    Per token: ``-(exp(logp − stop_grad(logp)) · A − β · k3(ref, logp))``; each sequence is averaged over its unmasked tokens and
    the batch over sequences.  The importance ratio is one by construction (a single policy update per batch of samples), so the
    clipping range ``epsilon`` is unused and the returned ``ratios`` / ``clipfrac`` are the constants 1 and 0.

    ``forward(pi_logits, targets, ref_logprobs, advantages, padding_masks)`` takes the logits whole or as a list of chunks along
    the sequence dimension (what a decoder with ``num_output_chunks`` set returns) and gives back
    ``(loss, policy_loss, kl_loss, ratios, clipfrac, pi_logprobs)``.
    """

    def __init__(self, num_output_chunks: int = 8, epsilon: float = 0.1, kl_coeff: float = 0.1):
        super().__init__()
        self.num_output_chunks, self.epsilon, self.kl_coeff = num_output_chunks, epsilon, kl_coeff

    def compute_per_token_quantities(self, pi_logits_chunk: torch.Tensor, targets_chunk: torch.Tensor, ref_logprobs_chunk: torch.Tensor, advantages: torch.Tensor):
        """One chunk ``[B·G, c, vocab]`` → per-token ``(loss, policy term, KL estimate, policy log-prob)``, each ``[B·G, c]``."""
        logp = torch.log_softmax(pi_logits_chunk.float(), dim=-1).gather(-1, targets_chunk.unsqueeze(-1)).squeeze(-1)
        kl = _k3(ref_logprobs_chunk.detach(), logp)
        policy = torch.exp(logp - logp.detach()) * advantages[:, None]
        return -(policy - self.kl_coeff * kl), policy, kl, logp

    def forward(self, pi_logits, targets: torch.Tensor, ref_logprobs: torch.Tensor, advantages: torch.Tensor, padding_masks: Optional[torch.Tensor] = None):
        chunks = [pi_logits] if isinstance(pi_logits, torch.Tensor) else list(pi_logits)
        keep = torch.ones_like(targets, dtype=torch.bool) if padding_masks is None else padding_masks
        n = len(chunks)
        sums = torch.zeros(3, advantages.numel(), device=chunks[0].device)  # per sequence: loss, policy, kl
        logps = []
        for logits, tgt, ref, m in zip(chunks, targets.chunk(n, dim=1), ref_logprobs.chunk(n, dim=1), keep.chunk(n, dim=1)):
            loss_t, policy_t, kl_t, logp = self.compute_per_token_quantities(logits, tgt, ref, advantages)
            m = m.to(loss_t.dtype)
            sums = sums + torch.stack([(loss_t * m).sum(1), (policy_t.detach() * m).sum(1), (kl_t.detach() * m).sum(1)])
            logps.append(logp)
        count = keep.sum(1).clamp(min=1e-9).to(sums.dtype)
        per_seq = (sums / count).mean(1)
        one = torch.ones((), device=sums.device)
        return per_seq[0], per_seq[1].detach(), per_seq[2].detach(), one, torch.zeros_like(one), torch.cat(logps, dim=1)
