# tune-recipe: distributed=false
"""Quantisation-aware full fine-tuning on one device.

    tune run qat_single_device --config <config> [key=value …]

Parity: recipes/qat_single_device.py of the reference (config keys ``quantizer``, ``fake_quant_after_n_steps``).
The loop is :class:`torchtune_b200.engine.qat.QATTrainer`; the quantisers are the package's own
(:mod:`torchtune_b200.training.quantization`).
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.qat import QATTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class QATRecipeSingleDevice(QATTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=False, lora=False)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="QATRecipeSingleDevice", cfg=cfg)
    recipe = QATRecipeSingleDevice(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
