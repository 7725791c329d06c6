"""AdamW whose two moments take one byte per parameter each.

The reference's low-memory single-device configs name ``bitsandbytes.optim.PagedAdamW8bit`` (e.g.
recipes/configs/llama3_1/8B_full_single_device.yaml:59-61) or ``torchao.optim.AdamW8bit``; neither package is part of this
framework, so the same idea is built in: block-wise quantised optimizer state.  Each block of 256 elements stores its largest
magnitude in fp32 and one code per element — the first moment as a signed code on a square-root scale, the second moment as an
unsigned code on a fourth-root scale, which puts the fine steps near zero where most entries of a block are (the two packages use
a non-uniform code table for the same reason).  The update itself is AdamW in fp32 (``torch.optim.AdamW`` semantics, decoupled
weight decay, bias correction).  State per parameter: 2 bytes + 1/32 byte, against 8 bytes for fp32 moments.

On CUDA one kernel per tensor expands, updates and re-codes (``ops/csrc/optim.cu::adamw8bit_kernel``); the statement of the same
arithmetic in PyTorch (``ops/reference.py::adamw8bit_step``) runs on CPU and is what the kernel is tested against.  Nothing is paged:
with 180 GB of device memory the state of the models this optimizer is meant for stays resident.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional, Tuple, Union

import torch
from torch.optim import Optimizer

from ..ops import reference as _ref


class AdamW8bit(Optimizer):
    def __init__(self, params: Iterable, lr: Union[float, torch.Tensor] = 1e-3, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 min_8bit_size: int = 4096, **ignored: Any):
        """``min_8bit_size``: tensors with fewer elements keep fp32 moments (norm scales, biases: tiny, and the most sensitive).
        Keyword arguments of the two packages' optimizers that have no meaning here (``block_size``, ``percentile_clipping``,
        ``is_paged``, ``bf16_stochastic_round`` …) are accepted and ignored."""
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("invalid AdamW hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, min_8bit_size=int(min_8bit_size)))
        self.grad_scale: Union[float, torch.Tensor] = 1.0

    def _init_state(self, p: torch.Tensor, group: Dict[str, Any]) -> Dict[str, Any]:
        st = self.state[p]
        if not st:
            st["step"] = 0
            n = p.numel()
            if n >= group["min_8bit_size"]:
                blocks = (n + _ref.ADAMW8BIT_BLOCK - 1) // _ref.ADAMW8BIT_BLOCK
                st["exp_avg_q"] = torch.zeros(n, dtype=torch.int8, device=p.device)
                st["exp_avg_sq_q"] = torch.zeros(n, dtype=torch.uint8, device=p.device)
                st["exp_avg_scale"] = torch.zeros(blocks, dtype=torch.float32, device=p.device)
                st["exp_avg_sq_scale"] = torch.zeros(blocks, dtype=torch.float32, device=p.device)
            else:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        return st

    def moments(self, p: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """fp32 ``(exp_avg, exp_avg_sq)`` of one parameter, expanded from the codes (for inspection and tests)."""
        st = self.state[p]
        if "exp_avg" in st:
            return st["exp_avg"].clone(), st["exp_avg_sq"].clone()
        m, v = _ref.adamw8bit_decode(st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"], p.numel())
        return m.view_as(p), v.view_as(p)

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for st in self.state.values() for t in st.values() if isinstance(t, torch.Tensor))

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """``torch.optim.Optimizer.load_state_dict`` casts every state tensor to its parameter's dtype, which would turn the codes
        into floats and round the fp32 scales of a bf16 parameter; the tensors are taken from ``state_dict`` again with their own
        dtypes."""
        super().load_state_dict(state_dict)
        ids = [pid for g in state_dict["param_groups"] for pid in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            for key, value in state_dict["state"].get(pid, {}).items():
                if isinstance(value, torch.Tensor) and key != "step":
                    self.state[p][key] = value.detach().clone().to(device=p.device)

    @torch.no_grad()
    def step(self, closure=None, grad_scale: Union[float, torch.Tensor, None] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        scale = self.grad_scale if grad_scale is None else grad_scale
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, eps, wd = float(group["lr"]), group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p, group)
                st["step"] += 1
                g = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                if "exp_avg" in st:
                    s = float(scale) if not isinstance(scale, float) else scale
                    w = p.detach().float()
                    _ref.adamw_step(w, g, st["exp_avg"], st["exp_avg_sq"], st["step"], lr, b1, b2, eps, wd, s)
                    p.copy_(w)
                    continue
                args = (st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"], st["step"], lr, b1, b2, eps, wd)
                if p.is_cuda and p.is_contiguous() and p.dtype in (torch.bfloat16, torch.float32) and g.dtype == p.dtype:
                    from ..ops import _cuda

                    _cuda.adamw8bit(p, g, *args, scale)
                else:
                    _ref.adamw8bit_step(p, g, *args, float(scale) if not isinstance(scale, float) else scale)
        return loss
