# tune-recipe: distributed=true
"""Quantisation-aware LoRA fine-tuning on N GPUs (fake-quantised base matmul, full-precision adapters).

    tune run --nproc_per_node 8 qat_lora_finetune_distributed --config <config> [key=value …]

Parity: recipes/qat_lora_finetune_distributed.py of the reference (config keys ``quantizer``, ``fake_quant_after_n_steps``).
The loop is :class:`torchtune_b200.engine.qat.QATTrainer`; the quantisers are the package's own
(:mod:`torchtune_b200.training.quantization`).
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.qat import QATTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class QATLoRAFinetuneRecipeDistributed(QATTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=True, lora=True)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="QATLoRAFinetuneRecipeDistributed", cfg=cfg)
    recipe = QATLoRAFinetuneRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
