# tune-recipe: distributed=false
"""Full-parameter supervised fine-tuning on one device.

    tune run full_finetune_single_device --config llama3_1/8B_full_single_device

Parity: recipes/full_finetune_single_device.py:124-718 of the reference (same config
keys); the training loop lives in :class:`torchtune_b200.engine.sft.SFTTrainer`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.sft import SFTTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class FullFinetuneRecipeSingleDevice(SFTTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=False, lora=False)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="FullFinetuneRecipeSingleDevice", cfg=cfg)
    recipe = FullFinetuneRecipeSingleDevice(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
