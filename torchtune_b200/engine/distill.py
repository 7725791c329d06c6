"""Knowledge distillation engine (student = LoRA or full model, teacher = frozen model).

Reference behaviour: recipes/knowledge_distillation_single_device.py:35-700 and
recipes/knowledge_distillation_distributed.py:40-900 — ``loss = (1 - kd_ratio)·CE +
kd_ratio·KD`` with ``class_loss`` / ``kd_loss`` logged beside ``loss``.

The student and teacher trunks return hidden states; both vocab projections and the two
losses are evaluated one sequence chunk at a time under recomputation, so only a single pair
of ``[chunk, vocab]`` fp32 logit blocks is alive at any point of forward or backward.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.utils.checkpoint import checkpoint

from .. import config, training, utils
from ..config import DictConfig
from .sft import SFTTrainer

log = utils.get_logger("DEBUG")


def _trunk(model: nn.Module, batch: Dict[str, Any]) -> torch.Tensor:
    core = getattr(model, "decoder", model)
    prev = getattr(core, "skip_output_layer", False)
    core.skip_output_layer = True
    try:
        out = model(**batch)
    finally:
        core.skip_output_layer = prev
    return out[-1] if isinstance(out, list) else out


class KDTrainer(SFTTrainer):
    def __init__(self, cfg: DictConfig, *, distributed: bool = False, lora: bool = True) -> None:
        super().__init__(cfg, distributed=distributed, lora=lora)
        self._kd_ratio = cfg.get("kd_ratio", 0.5)
        if self._optimizer_in_bwd:
            raise RuntimeError("optimizer_in_bwd is not supported by the knowledge-distillation recipes")

    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        super().setup(cfg)
        core = getattr(self._model, "decoder", self._model)
        core.skip_output_layer = False  # the engine switches it per call
        kd = config.instantiate(cfg.kd_loss)
        self._kd_loss_fn = getattr(kd, "inner", kd)  # chunked variants wrap a per-chunk divergence
        self._num_chunks = int(getattr(self._loss_fn, "num_output_chunks", 8) or 8)
        teacher_ckpt = config.instantiate(cfg.teacher_checkpointer, should_load_recipe_state=False).load_checkpoint()
        with training.set_default_dtype(self._dtype), self._device:
            teacher = config.instantiate(cfg.teacher_model)
        teacher.load_state_dict(teacher_ckpt[training.MODEL_KEY])
        teacher.eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        training.validate_expected_param_dtype(teacher.named_parameters(), dtype=self._dtype)
        self._teacher_model = teacher
        utils.log_rank_zero(log, "Teacher model is initialized.")

    def _chunk_losses(self, hs: torch.Tensor, ht: torch.Tensor, labels: torch.Tensor):
        s_logits = self._student_out(hs).float()
        with torch.no_grad():
            t_logits = self._teacher_out(ht).float()
        ignore = getattr(self._loss_fn, "ignore_index", -100)
        ce = F.cross_entropy(s_logits, labels, ignore_index=ignore, reduction="sum")
        kd = self._kd_loss_fn(s_logits, t_logits, labels, normalize=False)
        return ce, kd

    def _loss_step(self, batch: Dict[str, Any]):
        labels = batch.pop("labels")
        ignore = getattr(self._loss_fn, "ignore_index", -100)
        with self._activations_ctx:
            hs = _trunk(self._model, batch)
        with torch.no_grad():
            ht = _trunk(self._teacher_model, batch)
        # projection of already normalised hidden states, with whatever the decoder does to its logits (Gemma-2 soft cap)
        self._student_out = getattr(self._model, "decoder", self._model).unembed_normed
        self._teacher_out = getattr(self._teacher_model, "decoder", self._teacher_model).unembed_normed
        hs2, ht2, y = hs.reshape(-1, hs.shape[-1]), ht.reshape(-1, ht.shape[-1]), labels.reshape(-1)
        ce_sum = hs.new_zeros((), dtype=torch.float32)
        kd_sum = hs.new_zeros((), dtype=torch.float32)
        for a, b, c in zip(hs2.tensor_split(self._num_chunks), ht2.tensor_split(self._num_chunks), y.tensor_split(self._num_chunks)):
            if a.shape[0] == 0:
                continue
            if torch.is_grad_enabled():
                ce, kd = checkpoint(self._chunk_losses, a, b, c, use_reentrant=False)
            else:
                ce, kd = self._chunk_losses(a, b, c)
            ce_sum = ce_sum + ce
            kd_sum = kd_sum + kd
        n_valid = (y != ignore).sum()
        self._add_aux_sum("class_loss", ce_sum)
        self._add_aux_sum("kd_loss", kd_sum)
        return (1.0 - self._kd_ratio) * ce_sum + self._kd_ratio * kd_sum, n_valid
