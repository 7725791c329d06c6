# tune-recipe: distributed=false
"""LoRA / QLoRA / DoRA supervised fine-tuning on one device.

    tune run lora_finetune_single_device --config <config> [key=value …]

Parity: recipes/lora_finetune_single_device.py:46-760 of the reference (same config keys, metrics and checkpoint layout).
The loop is :class:`torchtune_b200.engine.sft.SFTTrainer`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.sft import SFTTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class LoRAFinetuneRecipeSingleDevice(SFTTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=False, lora=True)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="LoRAFinetuneRecipeSingleDevice", cfg=cfg)
    recipe = LoRAFinetuneRecipeSingleDevice(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
