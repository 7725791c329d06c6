# tune-recipe: distributed=true
"""Full fine-tuning with layer dropout and early-exit loss (LayerSkip, arXiv 2404.16710).

    tune run --nproc_per_node 8 dev/early_exit_finetune_distributed --config dev/7B_full_early_exit

Parity: recipes/dev/early_exit_finetune_distributed.py:40-1000 of the reference (config sections ``layer_dropout`` and
``early_exit_loss``).  The loop is :class:`torchtune_b200.engine.early_exit.EarlyExitTrainer`; every exit's loss goes
through the fused linear + cross-entropy operator.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.early_exit import EarlyExitTrainer
from torchtune_b200.recipe_interfaces import FTRecipeInterface
from torchtune_b200.utils import get_world_size_and_rank


class EarlyExitFinetuneRecipeDistributed(EarlyExitTrainer, FTRecipeInterface):
    def __init__(self, cfg: DictConfig) -> None:
        import os

        super().__init__(cfg, distributed=all(os.environ.get(k) for k in ("RANK", "WORLD_SIZE")), lora=False)


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="EarlyExitFinetuneRecipeDistributed", cfg=cfg)
    recipe = EarlyExitFinetuneRecipeDistributed(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.train()
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(recipe_main())
