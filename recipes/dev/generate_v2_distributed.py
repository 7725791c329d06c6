# tune-recipe: distributed=true
"""Tensor-parallel generation: the decoder's weights are split over all ranks, every rank decodes the same sequence.

    tune run --nproc_per_node 8 dev/generate_v2_distributed --config llama3_1/70B_generation_distributed
    tune run --nproc_per_node 8 dev/generate_v2_distributed --config llama4/scout_17B_16E_generation_distributed

Each rank keeps its slice of every projection (heads / MLP or expert columns) and its own KV cache; the two row-parallel
projections of a layer are summed over the ranks; all ranks sample with the same seed.  For an early-fusion model (Llama-4) the
vision encoder stays whole on every rank and only the decoder is split.  Same config surface as the reference's
recipes/dev/generate_v2_distributed.py; the work is done by :class:`torchtune_b200.engine.inference.SingleTurnGenerator`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.inference import SingleTurnGenerator


class InferenceRecipe(SingleTurnGenerator):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, tensor_parallel=True)


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="InferenceRecipe", cfg=cfg)
    recipe = InferenceRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.generate(cfg=cfg)
    recipe.cleanup()


if __name__ == "__main__":
    sys.exit(main())
