"""Optimizer stepped from inside backward (parity: torchtune/modules/optim.py:15-84)."""
from __future__ import annotations

from typing import Dict, Iterable, Type

import torch
from torch.optim import Optimizer


class OptimizerInBackward(Optimizer):
    """One inner optimizer per parameter, fired by that parameter's post-accumulate-grad
    hook, so a gradient is consumed and freed as soon as it is complete.  ``step()`` is a
    no-op by design."""

    def __init__(self, params: Iterable[torch.nn.Parameter], optimizer_cls: Type[Optimizer], **optimizer_kwargs):
        params = list(params)
        self._inner: Dict[int, Optimizer] = {}
        self._slot = {p: i for i, p in enumerate(params)}
        for i, p in enumerate(params):
            if not p.requires_grad:
                continue
            self._inner[i] = optimizer_cls([p], **optimizer_kwargs)
            p.register_post_accumulate_grad_hook(self._fire)
        super().__init__(params, optimizer_kwargs)

    def _fire(self, param: torch.nn.Parameter) -> None:
        opt = self._inner[self._slot[param]]
        opt.step()
        opt.zero_grad()

    def step(self, closure=None):
        if closure is not None:
            raise RuntimeError("OptimizerInBackward does not support closures.")

    def zero_grad(self, set_to_none: bool = True):
        for opt in self._inner.values():
            opt.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {
            "param_groups": super().state_dict()["param_groups"],
            "optimizers": {str(i): opt.state_dict() for i, opt in self._inner.items()},
            "state": {},
        }

    def load_state_dict(self, state_dict):
        super().load_state_dict({"param_groups": state_dict["param_groups"], "state": {}})
        for i, opt in self._inner.items():
            opt.load_state_dict(state_dict["optimizers"][str(i)])
