# tune-recipe: distributed=true
"""Knowledge distillation of a LoRA student from a frozen teacher on N GPUs.

    tune run --nproc_per_node 8 knowledge_distillation_distributed --config <config> [key=value …]

Parity: recipes/knowledge_distillation_distributed.py:40-900 of the reference (config keys ``teacher_model``,
``teacher_checkpointer``, ``kd_loss``, ``kd_ratio``; metrics ``loss``, ``class_loss``, ``kd_loss``).
The loop is :class:`torchtune_b200.engine.distill.KDTrainer`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.distill import KDTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface


class KDRecipeDistributed(KDTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, distributed=True, lora=cfg.model.get("lora_rank") is not None)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="KDRecipeDistributed", cfg=cfg)
    recipe = KDRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
