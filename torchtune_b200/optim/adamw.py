"""AdamW whose update is a single multi-tensor sm_100a kernel launch per dtype group.

Semantics follow ``torch.optim.AdamW`` (decoupled weight decay, bias correction, state
in the parameter dtype) as configured by the reference recipes
(recipes/configs/llama3_1/8B_full.yaml:66-69, ``fused: True``).  ``grad_scale`` lets the
caller fold gradient normalisation (÷ token count, clipping coefficient) into the update
instead of a separate pass over the gradients.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

import torch
from torch.optim import Optimizer

from ..ops import reference as _ref


class AdamW(Optimizer):
    def __init__(
        self,
        params: Iterable,
        lr: Union[float, torch.Tensor] = 1e-3,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
        fused: Optional[bool] = None,
        foreach: Optional[bool] = None,
        amsgrad: bool = False,
        master_weights: bool = False,
    ):
        if amsgrad:
            raise ValueError("amsgrad is not supported")
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("invalid AdamW hyper-parameters")
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, master_weights=master_weights)
        super().__init__(params, defaults)
        self.grad_scale: Union[float, torch.Tensor] = 1.0

    def _init_state(self, p: torch.Tensor, group: Dict[str, Any]) -> Dict[str, Any]:
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            if group["master_weights"] and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    @torch.no_grad()
    def step(self, closure=None, grad_scale: Union[float, torch.Tensor, None] = None, max_grad_norm: Optional[float] = None):
        """``grad_scale`` multiplies every gradient inside the update (float or 0-d device
        tensor, no host sync).  With ``max_grad_norm`` the global norm of the *scaled*
        gradients is clipped to it; the norm is returned as ``self.last_grad_norm``."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        scale = self.grad_scale if grad_scale is None else grad_scale
        self.last_grad_norm = None
        if max_grad_norm is not None:
            scale = self._clip_scale(scale, float(max_grad_norm))
        for group in self.param_groups:
            b1, b2 = group["betas"]
            cuda_items: List[Tuple[torch.Tensor, torch.Tensor, Dict[str, Any]]] = []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p, group)
                st["step"] += 1
                if p.is_cuda:
                    cuda_items.append((p, p.grad, st))
                else:
                    s = float(scale) if not isinstance(scale, float) else scale
                    _ref.adamw_step(p, p.grad, st["exp_avg"], st["exp_avg_sq"], st["step"], float(group["lr"]), b1, b2, group["eps"], group["weight_decay"], s, st.get("master"))
            if cuda_items:
                from ..ops import _cuda

                _cuda.adamw_multi(cuda_items, float(group["lr"]), b1, b2, group["eps"], group["weight_decay"], scale)
        return loss

    def _clip_scale(self, scale, max_norm: float):
        grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not grads:
            return scale
        if grads[0].is_cuda:
            from ..ops import _cuda

            items = [(p, p.grad, self._init_state(p, g)) for g in self.param_groups for p in g["params"] if p.grad is not None]
            sumsq = _cuda.grad_sumsq(items)
        else:
            sumsq = torch.stack([g.float().pow(2).sum() for g in grads]).sum()
        norm = sumsq.sqrt() * scale
        self.last_grad_norm = norm
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        return coef * scale
