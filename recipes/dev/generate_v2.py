# tune-recipe: distributed=false
"""Single-prompt generation for text and image+text models (deep- and early-fusion).

    tune run dev/generate_v2 --config llama2/generation_v2 prompt.user="Hello"

The prompt is one conversation turn given in the config (``prompt.system`` / ``prompt.user``; ``prompt.user`` may be
``{image: <path or url>, text: …}``).  Same config surface as the reference's recipes/dev/generate_v2.py; the work is done by
:class:`torchtune_b200.engine.inference.SingleTurnGenerator`.
"""
import sys

from torchtune_b200 import config
from torchtune_b200.config import DictConfig
from torchtune_b200.engine.inference import SingleTurnGenerator, prompt_to_messages


class InferenceRecipe(SingleTurnGenerator):
    def __init__(self, cfg: DictConfig) -> None:
        super().__init__(cfg, tensor_parallel=False)


# kept as an importable name for configs and scripts written against the reference recipe
class SingleTurnYAMLToMessages:
    def __call__(self, prompt):
        return prompt_to_messages(prompt)


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="InferenceRecipe", cfg=cfg)
    recipe = InferenceRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.generate(cfg=cfg)


if __name__ == "__main__":
    sys.exit(main())
