"""GRPO objective fused with the output projection (parity: torchtune/dev/rl/linear_grpo_loss.py:17-182).

The policy's per-token log-probabilities come straight from the hidden states through :func:`torchtune_b200.ops.token_logprobs`:
on CUDA that is the chunked tcgen05 projection + in-place softmax kernel pair (``ops/csrc/loss.cu``), whose backward recomputes each
logits chunk, so neither the ``[tokens, vocab]`` logits nor their fp32 log-softmax ever exist in full — the reference reaches the
same memory picture by chunking ``F.cross_entropy`` in Python.  What remains is element-wise work on ``[B·G, L]`` log-probabilities:

    per token  loss = −( exp(logp − stop_grad(logp)) · A  −  β · k3 ),   k3 = exp(ref − logp) − (ref − logp) − 1

averaged over each sequence's unmasked tokens, then over sequences.  One policy update is made per batch of samples, so the
importance ratio is 1 by construction and ``epsilon`` (kept for config parity) is unused."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ... import ops


class LinearGRPOLoss(nn.Module):
    def __init__(self, num_output_chunks: int = 8, epsilon: float = 0.1, kl_coeff: float = 0.1, ignore_index: int = -100, mask_pre_projection: bool = True):
        super().__init__()
        self.linear_projection = None
        self.num_output_chunks, self.epsilon, self.kl_coeff, self.ignore_index, self.mask_pre_projection = num_output_chunks, epsilon, kl_coeff, ignore_index, mask_pre_projection

    def apply_compile_strategy(self, *args, **kwargs):
        return self  # nothing to trace: the projection and the softmax are kernels already

    def set_model_output(self, model: nn.Module) -> None:
        model.skip_output_layer = True
        self.linear_projection = model.output
        self.logit_softcap = ops.logit_softcap_of(model)

    def _weight(self) -> torch.Tensor:
        proj = self.linear_projection
        if proj is None:
            raise RuntimeError("call set_model_output(model) before the loss")
        weight = getattr(proj, "weight", None)
        if weight is None and hasattr(proj, "tied_module"):
            weight = proj.tied_module.weight
        if weight is None:
            raise TypeError("the output projection has no weight matrix")
        return weight

    def forward(self, pi_old_outputs: torch.Tensor, pi_outputs: torch.Tensor, ref_outputs: torch.Tensor, advantages: torch.Tensor,
                padding_masks: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, ...]:
        """``pi_old_outputs``: hidden states ``[B·G, L, dim]`` (before the output projection); ``pi_outputs``: target tokens
        ``[B·G, L]``; ``ref_outputs``: reference log-probabilities ``[B·G, L]``; ``advantages`` ``[B·G]``; ``padding_masks`` ``[B·G, L]``
        True = token counts.  Returns ``(loss, policy_loss, kl_loss, ratios, clipfrac, pi_logprobs)``."""
        keep = torch.ones_like(pi_outputs, dtype=torch.bool) if padding_masks is None else padding_masks
        targets = pi_outputs
        if self.mask_pre_projection:  # ignored positions cost no softmax work and get a log-probability of exactly zero
            targets = torch.where(keep, pi_outputs, torch.full_like(pi_outputs, self.ignore_index))
        logp = ops.token_logprobs(pi_old_outputs, self._weight(), targets, ignore_index=self.ignore_index, num_chunks=self.num_output_chunks,
                                  softcap=getattr(self, "logit_softcap", 0.0)).float()
        ref = ref_outputs.detach().float()
        d = ref - logp
        kl = torch.exp(d) - d - 1
        policy = torch.exp(logp - logp.detach()) * advantages.float()[:, None]
        per_token = -(policy - self.kl_coeff * kl)
        m = keep.to(per_token.dtype)
        count = m.sum(1).clamp(min=1e-9)
        loss = ((per_token * m).sum(1) / count).mean()
        with torch.no_grad():
            policy_loss = ((policy * m).sum(1) / count).mean()
            kl_loss = ((kl * m).sum(1) / count).mean()
        one = torch.ones((), device=loss.device)
        return loss, policy_loss, kl_loss, one, torch.zeros_like(one), logp.detach()
