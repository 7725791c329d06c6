# tune-recipe: distributed=false
"""Asynchronous GRPO: inference, post-processing and training run as concurrent roles that exchange trajectories and weights.

    tune run dev/async_grpo_full_finetune_distributed --config dev/qwen3B_async_grpo

This launches only the controller (no ``--nproc_per_node``): it builds the roles, places them on the visible GPUs and runs them
until the trainer has made ``orchestration.num_steps`` steps.  Parity: recipes/dev/async_grpo_full_finetune_distributed.py:118-315
(config sections ``orchestration``, ``inference``, ``postprocessing``, ``training``, ``reward_functions``).  The controller is
:class:`torchtune_b200.engine.async_grpo.AsyncGRPORecipe`; the roles live in :mod:`torchtune_b200.dev.rl.workers`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.async_grpo import AsyncGRPORecipe


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="AsyncGRPORecipe", cfg=cfg)
    recipe = AsyncGRPORecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    try:
        recipe.train()
    finally:
        recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
