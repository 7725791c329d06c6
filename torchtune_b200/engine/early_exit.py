"""Early-exit (LayerSkip) fine-tuning engine: layer dropout + early-exit loss with a curriculum
(reference behaviour: recipes/dev/early_exit_finetune_distributed.py:40-1000; arXiv 2404.16710).

Config sections (both optional): ``layer_dropout: {prob, layers, layers_scale, disable_on_eval}`` and
``early_exit_loss: {layers, curriculum, scale_fn, scale, include_last_layer, verbose}``."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .. import utils
from ..config import DictConfig
from ..config._resolve import get_component_from_path
from ..modules.common_utils import slice_str_to_array
from ..modules.early_exit_loss import early_exit_loss
from ..modules.layer_dropout import prepare_layer_dropout
from .sft import SFTTrainer

log = utils.get_logger("DEBUG")


class EarlyExitTrainer(SFTTrainer):
    def __init__(self, cfg: DictConfig, *, distributed: bool = True, lora: bool = False) -> None:
        super().__init__(cfg, distributed=distributed, lora=lora)
        ee = cfg.get("early_exit_loss")
        self._do_early_exit = bool(ee)
        self._ee_scale = ee.get("scale", 1.0) if ee else None
        self._ee_scale_fn = get_component_from_path(ee.get("scale_fn", "torchtune_b200.modules.early_exit_loss.sum_l_loss_scale")) if ee else None
        self._curriculum = None

    def _transform_model(self, model, cfg: DictConfig):
        model = super()._transform_model(model, cfg)
        ld = cfg.get("layer_dropout")
        if ld:
            prepare_layer_dropout(model.layers, prob_max=ld.get("prob", 0.0), prob_layer_scale=ld.get("layers_scale", "uniform"), layers_str=ld.get("layers", ":"), disable_on_eval=ld.get("disable_on_eval", True))
        return model

    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        super().setup(cfg)
        ee = cfg.get("early_exit_loss")
        if not ee:
            return
        core = getattr(self._model, "decoder", self._model)
        core.skip_output_layer = True  # every exit (including the last) goes through the fused linear-CE operator
        n_layers = len(core.layers)
        active = slice_str_to_array(ee.get("layers", ":"), n_layers)
        curriculum = ee.get("curriculum")
        if curriculum:
            cls = get_component_from_path(curriculum)
            self._curriculum = cls(do_output_hidden_states=active, max_steps=self.total_training_steps, train_last_layer=ee.get("include_last_layer", True),
                                   last_step=self.global_step, verbose=ee.get("verbose", False))
            active = self._curriculum.get()
        self._set_exits(active)

    def _set_exits(self, active) -> None:
        core = getattr(self._model, "decoder", self._model)
        core.output_hidden_states = [i for i, on in enumerate(active) if on]

    def _loss_step(self, batch: Dict[str, Any]):
        if not self._do_early_exit:
            return super()._loss_step(batch)
        core = getattr(self._model, "decoder", self._model)
        labels = batch.pop("labels")
        ignore = getattr(self._loss_fn, "ignore_index", -100)
        n_valid = (labels != ignore).sum()
        with self._activations_ctx:
            outputs = self._model(**batch)
        if core.output_hidden_states:
            final = outputs[-1]
            hidden = {i: h for i, h in zip(core.output_hidden_states, outputs[:-1])}
            # hidden state i is the input of layer i; the model output (already normalised) is exit `n_layers`
            loss = early_exit_loss(core, hidden, labels, self._loss_fn, self._ee_scale, self._ee_scale_fn) if hidden else 0.0
            last_sum, _ = self._loss_fn.compute_sum(final, labels)
            if hidden:
                ids = torch.tensor(list(hidden.keys()) + [len(core.layers) - 1], dtype=torch.float32, device=labels.device)
                scales = self._ee_scale_fn(ids, len(core.layers), self._ee_scale)
                # re-weight: early exits share (1 - w_last), the final layer takes w_last
                w_last = scales[-1]
                loss = (1.0 - w_last) * loss + w_last * last_sum / n_valid.clamp_min(1)
            else:
                loss = last_sum / n_valid.clamp_min(1)
            return loss * n_valid, n_valid
        total, _ = self._loss_fn.compute_sum(outputs, labels)
        return total, n_valid

    def _after_step(self) -> None:
        if self._curriculum is not None:
            self._curriculum.step()
            self._set_exits(self._curriculum.get())
