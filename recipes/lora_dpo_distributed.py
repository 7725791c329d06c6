# tune-recipe: distributed=true
"""LoRA direct preference optimisation on N GPUs (reference model = adapters switched off).

    tune run --nproc_per_node 8 lora_dpo_distributed --config <config> [key=value …]

Parity: recipes/lora_dpo_distributed.py:47-800 of the reference (same config keys, logged metrics and checkpoint
layout).  The loop is :class:`torchtune_b200.engine.preference.DPOTrainer`: sequence
log-probabilities come from the fused hidden→log-prob operator, so no ``[2B, L, vocab]``
logits tensor is materialised for either the policy or the reference pass.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.preference import DPOTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class LoRADPORecipeDistributed(DPOTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=True, lora=True)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="LoRADPORecipeDistributed", cfg=cfg)
    recipe = LoRADPORecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
