"""Preference losses (parity: torchtune/rlhf/loss/dpo.py:17-181)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .._types import ChosenRejectedOutputs


def _margin(policy: ChosenRejectedOutputs, reference: ChosenRejectedOutputs) -> torch.Tensor:
    return (policy.chosen_logps - policy.rejected_logps) - (reference.chosen_logps - reference.rejected_logps)


def _implicit_rewards(scale: float, policy: ChosenRejectedOutputs, reference: ChosenRejectedOutputs):
    return scale * (policy.chosen_logps - reference.chosen_logps).detach(), scale * (policy.rejected_logps - reference.rejected_logps).detach()


class PreferenceLoss(nn.Module):
    def is_reference_free(self) -> bool:
        return False


class DPOLoss(PreferenceLoss):
    """Direct Preference Optimization (arXiv 2305.18290):
    ``-(1-ε)·logσ(β·Δ) - ε·logσ(-β·Δ)`` with ``Δ`` the policy-minus-reference log-ratio margin
    and ``ε`` the label smoothing.  Returns per-example losses and the implicit rewards."""

    def __init__(self, beta: float = 0.1, label_smoothing: float = 0.0):
        super().__init__()
        self.beta = beta
        self.label_smoothing = label_smoothing

    def forward(self, policy_inputs: ChosenRejectedOutputs, reference_inputs: ChosenRejectedOutputs) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        delta = _margin(policy_inputs, reference_inputs)
        losses = -F.logsigmoid(self.beta * delta) * (1 - self.label_smoothing) - F.logsigmoid(-self.beta * delta) * self.label_smoothing
        return (losses, *_implicit_rewards(self.beta, policy_inputs, reference_inputs))


class RSOLoss(PreferenceLoss):
    """Statistical Rejection Sampling Optimization (arXiv 2309.06657): hinge loss
    ``relu(1 - γ·Δ)`` on the same margin."""

    def __init__(self, gamma: float = 0.1):
        super().__init__()
        self.gamma = gamma

    def forward(self, policy_inputs: ChosenRejectedOutputs, reference_inputs: ChosenRejectedOutputs) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        losses = torch.relu(1 - self.gamma * _margin(policy_inputs, reference_inputs))
        return (losses, *_implicit_rewards(self.gamma, policy_inputs, reference_inputs))
