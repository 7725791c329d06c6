# tune-recipe: distributed=true
"""GRPO (group-relative policy optimisation) full fine-tuning, synchronous, on one or N GPUs.

    tune run --nproc_per_node 8 dev/grpo_full_finetune_distributed --config dev/3B_full_grpo

Parity: recipes/dev/grpo_full_finetune_distributed.py:60-1100 of the reference (config keys ``grpo_samples``, ``batch_size``,
``forward_batch_size``, ``max_generated_tokens``, ``temperature``, ``top_k``, ``ppo_epochs``, ``num_steps``, ``ref_checkpointer``,
``loss``, optional ``reward_fn``).  The loop is :class:`torchtune_b200.engine.grpo.GRPOTrainer`.
"""
import os
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.grpo import GRPOTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class GRPOFullFinetuneRecipeDistributed(GRPOTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=all(os.environ.get(k) for k in ("RANK", "WORLD_SIZE")))

    def load_checkpoint(self, **kwargs):
        raise NotImplementedError("use setup(); this recipe reads the policy and the reference checkpoints together")


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="GRPOFullFinetuneRecipeDistributed", cfg=cfg)
    recipe = GRPOFullFinetuneRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
