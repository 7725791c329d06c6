# tune-recipe: distributed=false
"""Proximal policy optimisation (RLHF) of a policy and value model on one device.

    tune run ppo_full_finetune_single_device --config mistral/7B_full_ppo_low_memory [key=value …]

Parity: recipes/ppo_full_finetune_single_device.py:38-1240 of the reference (same config keys:
``policy_model``, ``reward_and_value_model``, the four checkpointers, ``num_steps``,
``forward_batch_size``, ``ppo_batch_size``, ``ppo_epochs``, ``kl_coeff``, ``gamma``, ``lmbda`` …;
same logged metrics).  The loop is :class:`torchtune_b200.engine.ppo.PPOTrainer`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.ppo import PPOTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class PPOFullFinetuneRecipeSingleDevice(PPOTrainer, FTRecipeInterface):
    def load_checkpoint(self, **kwargs):  # checkpoints are read inside setup(): four of them
        raise NotImplementedError("use setup(); this recipe reads policy, reference, value and reward checkpoints together")


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="PPOFullFinetuneRecipeSingleDevice", cfg=cfg)
    recipe = PPOFullFinetuneRecipeSingleDevice(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
