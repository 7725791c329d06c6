"""Quantisation-aware training engine (full and LoRA).

Reference behaviour: recipes/qat_single_device.py, recipes/qat_distributed.py:60-1100 (a
``quantizer`` config entry whose ``prepare`` inserts fake quantisation; optional
``fake_quant_after_n_steps`` warm-up in full precision) and
recipes/qat_lora_finetune_distributed.py:60-1000 (LoRA layers swapped for QAT-LoRA layers,
adapters stay in full precision).  The saved checkpoint holds ordinary full-precision
weights; ``tune run quantize`` with the matching post-training quantiser converts them.
"""
from __future__ import annotations

from typing import Optional

from torch import nn

from .. import config, training, utils
from ..config import DictConfig
from ..training import quantization as Q
from .sft import SFTTrainer

log = utils.get_logger("DEBUG")


class QATTrainer(SFTTrainer):
    def __init__(self, cfg: DictConfig, *, distributed: bool = False, lora: bool = False) -> None:
        super().__init__(cfg, distributed=distributed, lora=lora)
        self._fake_quant_after_n_steps: Optional[int] = cfg.get("fake_quant_after_n_steps")
        self._quantizer_mode: Optional[str] = None

    def _transform_model(self, model: nn.Module, cfg: DictConfig) -> nn.Module:
        model = super()._transform_model(model, cfg)
        if self.is_lora:
            qcfg = cfg.get("quantizer")
            group = (qcfg.get("groupsize") if qcfg is not None else None) or 256
            act = Q.FakeQuantizeConfig(bits=8, group_size=None, is_symmetric=False)
            wt = Q.FakeQuantizeConfig(bits=4, group_size=group, is_symmetric=True)
            Q.swap_lora_linear_with_qat(model, act, wt)
            self._quantizer_mode = "8da4w-qat"
            return model
        if cfg.get("quantizer") is None:
            raise ValueError("Quantizer must be specified for QAT recipe.")
        quantizer = config.instantiate(cfg.quantizer)
        mode = Q.get_quantizer_mode(quantizer)
        if mode is None or "qat" not in mode:
            raise ValueError("Quantizer mode '%s' is not supported for finetuning" % mode)
        self._quantizer_mode = mode
        model = quantizer.prepare(model)
        if self._fake_quant_after_n_steps is not None:
            model.apply(Q.disable_fake_quant)
        return model

    def _before_batch(self, idx: int) -> None:
        n = self._fake_quant_after_n_steps
        if n is None:
            return
        if self.global_step == 0 and idx == 0:
            utils.log_rank_zero(log, f"Step 0: Disabling fake quant, will re-enable in step {n}")
            self._model.apply(Q.disable_fake_quant)
        elif self.global_step == n and not getattr(self, "_fq_enabled", False):
            utils.log_rank_zero(log, f"Step {n}: Enabling fake quant")
            self._model.apply(Q.enable_fake_quant)
            self._fq_enabled = True
