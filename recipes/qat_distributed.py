# tune-recipe: distributed=true
"""Quantisation-aware full fine-tuning on N GPUs.

    tune run --nproc_per_node 8 qat_distributed --config <config> [key=value …]

Parity: recipes/qat_distributed.py of the reference (config keys ``quantizer``, ``fake_quant_after_n_steps``).
The loop is :class:`torchtune_b200.engine.qat.QATTrainer`; the quantisers are the package's own
(:mod:`torchtune_b200.training.quantization`).
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.qat import QATTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class QATRecipeDistributed(QATTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=True, lora=False)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="QATRecipeDistributed", cfg=cfg)
    recipe = QATRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
