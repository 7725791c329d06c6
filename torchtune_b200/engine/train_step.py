"""One optimisation step as a callable: host batch in, loss out.

``TrainStep`` is the smallest public unit a user drives directly (the recipes' loops are
built from the same pieces): it uploads a batch from (pinned) host memory, runs forward and
backward through the sm_100a kernels, normalises by the global number of unmasked label
tokens, steps the optimizer and returns the mean token loss as a device scalar — the
caller decides when to synchronise (``.item()``).

Token accounting follows the reference recipes: the summed loss is back-propagated and the
gradients are divided by the all-reduced token count inside the optimizer update
(recipes/full_finetune_distributed.py:1007-1039).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
from torch import nn

from ..ops.mask import AttentionMask
from ..utils import batch_to_device


class TrainStep:
    def __init__(self, model: nn.Module, loss_fn, optimizer, device: torch.device, parallel=None, clip_grad_norm: Optional[float] = None):
        self.model, self.loss_fn, self.optimizer = model, loss_fn, optimizer
        self.device = device
        self.parallel = parallel
        self.clip_grad_norm = clip_grad_norm
        self._params = [p for p in model.parameters() if p.requires_grad]

    def upload(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        out = dict(batch)
        batch_to_device(out, self.device)
        return out

    def compute(self, batch: Dict[str, Any]) -> torch.Tensor:
        """Forward, backward and update on a batch that already lives on the device."""
        batch = dict(batch)
        labels = batch.pop("labels")
        hidden = self.model(**batch)
        loss_sum, n_valid = self.loss_fn.compute_sum(hidden, labels)
        n_tokens = n_valid.to(torch.float32)
        if self.parallel is not None:
            # the global token count is known before backward, so the optimizer can consume each layer's gradients while
            # backward is still running on the earlier layers
            total = loss_sum.detach().clone()
            self.parallel.all_reduce_sum_(n_tokens, total)
            scale = 1.0 / n_tokens
            if hasattr(self.parallel, "arm_backward_overlap"):
                self.parallel.arm_backward_overlap(self.optimizer, scale, self.clip_grad_norm)
            loss_sum.backward()
            self.parallel.optimizer_step(self.model, self.optimizer, scale, self.clip_grad_norm)
            return total / n_tokens
        loss_sum.backward()
        self.optimizer.step(grad_scale=1.0 / n_tokens, max_grad_norm=self.clip_grad_norm)
        self.optimizer.zero_grad(set_to_none=True)
        return loss_sum.detach() / n_tokens

    def __call__(self, host_batch: Dict[str, Any]) -> torch.Tensor:
        return self.compute(self.upload(host_batch))
