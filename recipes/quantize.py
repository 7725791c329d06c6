# tune-recipe: distributed=false
"""Post-training quantisation of a checkpoint.

    tune run quantize --config quantization

Parity: recipes/quantize.py:24-140 of the reference.  ``quantizer`` is one of the package's
quantisers (:mod:`torchtune_b200.training.quantization`): a post-training one
(``Int8DynActInt4WeightQuantizer``, ``Int4WeightOnlyQuantizer``) or, for a model trained with
QAT, the matching QAT quantiser (prepare + convert).  The output is
``<output_dir>/<first checkpoint file stem>-<mode>.pt``.
"""
import os
import sys
import time
from pathlib import Path
from typing import Any, Dict

import torch

from torchtune_b200 import config, training, utils
from torchtune_b200.config import DictConfig

logger = utils.get_logger("DEBUG")


class QuantizationRecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self._device)
        self._quantizer = config.instantiate(cfg.quantizer)
        self._quantization_mode = training.get_quantizer_mode(self._quantizer)
        if self._quantization_mode is None:
            raise ValueError(f"Quantizer {type(self._quantizer).__name__} is not supported.")
        training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))

    def load_checkpoint(self, checkpointer_cfg: DictConfig) -> Dict[str, Any]:
        self._checkpointer = config.instantiate(checkpointer_cfg)
        return self._checkpointer.load_checkpoint()

    def setup(self, cfg: DictConfig) -> None:
        ckpt = self.load_checkpoint(cfg.checkpointer)
        with training.set_default_dtype(self._dtype), self._device:
            model = config.instantiate(cfg.model)
        if "qat" in self._quantization_mode:
            model = self._quantizer.prepare(model)
        model.load_state_dict(ckpt[training.MODEL_KEY])
        self._model = model
        logger.info(f"Model is initialized with precision {self._dtype}.")

    @torch.no_grad()
    def quantize(self, cfg: DictConfig) -> None:
        t0 = time.perf_counter()
        if "qat" in self._quantization_mode:
            self._model = self._quantizer.convert(self._model)
        else:
            self._model = self._quantizer.quantize(self._model)
        logger.info(f"Time for quantization: {time.perf_counter() - t0:.02f} sec")
        if self._device.type == "cuda":
            logger.info(f"Memory used: {torch.cuda.max_memory_allocated(self._device) / 1e9:.02f} GB")

    def save_checkpoint(self, cfg: DictConfig) -> None:
        files = cfg.checkpointer.checkpoint_files
        first = files[0] if not hasattr(files, "get") or files.get("filename_format") is None else files.get("filename_format")
        stem = Path(str(first)).stem
        out_dir = Path(cfg.checkpointer.output_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        out = out_dir / f"{stem}-{self._quantization_mode}.pt"
        torch.save({k: v.cpu() for k, v in self._model.state_dict().items()}, out)
        logger.info(f"Model checkpoint of size {os.path.getsize(out) / 1024**2:.2f} MiB saved to {out}")


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="QuantizationRecipe", cfg=cfg)
    recipe = QuantizationRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.quantize(cfg=cfg)
    recipe.save_checkpoint(cfg=cfg)


if __name__ == "__main__":
    sys.exit(main())
