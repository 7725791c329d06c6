# tune-recipe: distributed=true
"""Full-parameter supervised fine-tuning on N GPUs (one process per GPU).

    tune run --nproc_per_node 8 full_finetune_distributed --config <config> [key=value …]

Parity: recipes/full_finetune_distributed.py:53-1169 of the reference (same config keys, metrics and checkpoint layout).
The loop is :class:`torchtune_b200.engine.sft.SFTTrainer`; gradients and parameters move through
the resident data-parallel engine (flat peer buffers, one fused reduce→AdamW→broadcast kernel
per step) instead of per-layer FSDP collectives.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.sft import SFTTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class FullFinetuneRecipeDistributed(SFTTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=True, lora=False)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="FullFinetuneRecipeDistributed", cfg=cfg)
    recipe = FullFinetuneRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
