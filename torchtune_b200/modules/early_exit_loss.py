"""Early-exit (LayerSkip) loss and curricula (parity: torchtune/modules/early_exit_loss.py:19-290).

The loss un-embeds the hidden states of selected layers with the shared output head and adds their
cross-entropies with per-layer weights; a curriculum decides, step by step, which layers take part.
The per-layer losses go through the fused linear+cross-entropy operator, so no ``[layers, tokens, vocab]``
logits tensor is materialised."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .. import ops, utils

log = utils.get_logger("DEBUG")


def _finish(scales: torch.Tensor, layer_ids: torch.Tensor, n_layers: int, e_scale: float) -> torch.Tensor:
    scales = scales * torch.where(layer_ids < n_layers - 1, e_scale, 1.0)  # the last layer is never down-weighted
    return scales / scales.sum()


def uniform_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(torch.ones(len(layer_ids), device=layer_ids.device), layer_ids, n_layers, e_scale)


def linear_l_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(layer_ids + 1.0, layer_ids, n_layers, e_scale)


def sum_l_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(torch.cumsum(layer_ids + 1.0, dim=0), layer_ids, n_layers, e_scale)


def sqrt_l_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(torch.sqrt(layer_ids + 1.0), layer_ids, n_layers, e_scale)


def inv_l_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(1.0 / (layer_ids + 1.0), layer_ids, n_layers, e_scale)


def inv_sqrt_l_loss_scale(layer_ids: torch.Tensor, n_layers: int, e_scale: float = 1.0) -> torch.Tensor:
    return _finish(torch.rsqrt(layer_ids + 1.0), layer_ids, n_layers, e_scale)


def early_exit_loss(model, hidden_states_dict: Dict[int, torch.Tensor], labels: torch.Tensor, loss_fn: torch.nn.Module, e_scale: float = 1.0,
                    loss_scale_fn: Callable[[torch.Tensor, int, float], torch.Tensor] = uniform_loss_scale) -> torch.Tensor:
    """``Σ_l w_l · CE(unembed(h_l), labels)`` over the layers in ``hidden_states_dict`` (layer index → hidden state);
    every CE is normalised by the number of un-ignored labels."""
    ignore = getattr(loss_fn, "ignore_index", -100)
    ids = list(hidden_states_dict.keys())
    weight = model.output.weight if hasattr(model.output, "weight") else model.output.tied_module.weight
    n_valid = (labels != ignore).sum().clamp_min(1)
    losses = []
    for h in hidden_states_dict.values():
        total, _ = ops.linear_cross_entropy(model.norm(h), weight, labels, ignore_index=ignore, num_chunks=8, softcap=ops.logit_softcap_of(model))
        losses.append(total.float() / n_valid)
    losses = torch.stack(losses)
    scales = loss_scale_fn(torch.tensor(ids, dtype=torch.float32, device=losses.device), len(model.layers), e_scale)
    return torch.sum(scales * losses)


class EarlyExitCurriculum:
    """Decides which layers emit hidden states for the early-exit loss at the current step."""

    def __init__(self, do_output_hidden_states: List[bool], max_steps: int, train_last_layer: bool = True, last_step: Optional[int] = None, verbose: bool = False):
        self._init_do_output_hidden_states = do_output_hidden_states
        self._do_output_hidden_states = np.array(do_output_hidden_states, dtype=bool)
        self.train_last_layer, self.verbose, self.max_steps = train_last_layer, verbose, max_steps
        self._step = 0 if last_step is None else last_step

    def step(self) -> None:
        pass

    def get(self) -> np.ndarray:
        out = np.copy(self._do_output_hidden_states)
        if self.train_last_layer:
            out[-1] = True
        return out


class RotationalEarlyExitCurriculum(EarlyExitCurriculum):
    """The set of active layers shifts by one layer every step (wrapping around)."""

    def step(self) -> None:
        self._do_output_hidden_states = np.roll(self._do_output_hidden_states, 1)
        self._step += 1
        if self.verbose:
            log.info(f"Updated self._do_output_hidden_states to {self._do_output_hidden_states}.")


class GradualEarlyExitCurriculum(EarlyExitCurriculum):
    """Layers are switched on from the last towards the first as training progresses: layer ``l`` of ``n`` joins once
    the fraction of completed steps reaches ``fraction_scale · (n - l) / n``."""

    def __init__(self, do_output_hidden_states: List[bool], max_steps: int, train_last_layer: bool = True, last_step: Optional[int] = None, fraction_scale: float = 0.5, verbose: bool = False):
        super().__init__(do_output_hidden_states, max_steps, train_last_layer, last_step, verbose)
        self._final_do_output_hidden_states = np.copy(self._do_output_hidden_states)
        self._step = 0
        self._fraction_scale = fraction_scale
        self._do_output_hidden_states = np.zeros_like(self._final_do_output_hidden_states)

    def step(self) -> None:
        done = self._step / self.max_steps
        n = len(self._final_do_output_hidden_states)
        reached = np.array([done >= self._fraction_scale * (n - l) / n for l in range(n)])
        self._do_output_hidden_states = np.logical_and(reached, self._final_do_output_hidden_states)
        self._step += 1
        if self.verbose:
            log.info(f"Updated self._do_output_hidden_states to {self._do_output_hidden_states}.")
