"""Fused output-projection + cross-entropy (parity: torchtune/modules/loss/cross_entropy_loss.py:19-188)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ... import ops
from .loss_types import SFTLoss


class LinearCrossEntropyLoss(nn.Module, SFTLoss):
    """Mean token cross entropy computed from *hidden states*.

    ``set_model_output(model)`` flips ``model.skip_output_layer`` and keeps a handle to
    ``model.output``; ``forward(hidden, targets)`` then applies the projection chunk by
    chunk inside :func:`torchtune_b200.ops.linear_cross_entropy`, so the ``[tokens,
    vocab]`` logits never exist in memory.  Ignored targets do not contribute; with no
    valid target the loss is 0.
    """

    def __init__(self, num_output_chunks: int = 8, ignore_index: int = -100, tp_enabled: bool = False, mask_ignored_tokens: bool = True):
        super().__init__()
        self.linear_projection: Optional[nn.Module] = None
        self.num_output_chunks = num_output_chunks
        self.ignore_index = ignore_index
        self.tp_enabled = tp_enabled
        self.mask_ignored_tokens = mask_ignored_tokens
        self.logit_softcap = 0.0

    def set_model_output(self, model: nn.Module) -> None:
        model.skip_output_layer = True
        self.linear_projection = model.output
        self.logit_softcap = ops.logit_softcap_of(model)  # a fusion model keeps the cap on its decoder

    def patch_tp_plan(self, tp_plan) -> dict:
        self.tp_enabled = True
        return tp_plan

    @property
    def tp_requires_loss_parallel_ctx_manager(self) -> bool:
        return True

    def _weight(self) -> torch.Tensor:
        if self.linear_projection is None:
            raise AttributeError("forward called before update_model")
        return self.linear_projection.weight

    def compute_sum(self, outputs: torch.Tensor, targets: torch.Tensor):
        """``(sum of token losses, number of valid tokens)`` — what distributed recipes
        need for global token normalisation."""
        proj = self.linear_projection
        if self.logit_softcap > 0.0:
            # Gemma-2: the cap sits between the projection and the softmax; the fused op applies it inside its softmax kernel
            if proj is not None and hasattr(proj, "linear_cross_entropy"):
                raise NotImplementedError("soft-capped logits with a sharded output projection")
            return ops.linear_cross_entropy(outputs, self._weight(), targets, self.ignore_index, self.num_output_chunks, softcap=self.logit_softcap)
        if proj is not None and hasattr(proj, "linear_cross_entropy"):
            # sharded / tensor-parallel projections own their fused loss
            return proj.linear_cross_entropy(outputs, targets, self.ignore_index, self.num_output_chunks)
        return ops.linear_cross_entropy(outputs, self._weight(), targets, self.ignore_index, self.num_output_chunks)

    def forward(self, outputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        total, n_valid = self.compute_sum(outputs, targets)
        if isinstance(n_valid, torch.Tensor):
            return total / n_valid.clamp_min(1).to(total.dtype)
        return total / max(n_valid, 1)
