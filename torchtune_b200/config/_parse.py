"""``@config.parse`` decorator and its argument parser (parity: torchtune/config/_parse.py:20-101)."""
from __future__ import annotations

import argparse
import functools
import sys
from typing import Any, Callable, List, Tuple

from ._node import DictConfig, OmegaConf
from ._utils import _merge_yaml_and_cli_args

Recipe = Callable[[DictConfig], Any]


class TuneRecipeArgumentParser(argparse.ArgumentParser):
    """Parser whose defaults come from the YAML file named by ``--config``.

    Everything that is not a known flag is returned untouched as the override
    list; unknown ``--flags`` are an error.
    """

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        super().add_argument("--config", type=str, help="Path/name of a yaml file with configurations", required=True)

    def parse_known_args(self, *args, **kwargs) -> Tuple[argparse.Namespace, List[str]]:
        namespace, rest = super().parse_known_args(*args, **kwargs)
        flags = [a for a in rest if a.startswith("--")]
        if flags:
            raise ValueError(f"Additional flag arguments not supported: {flags}. Please use --config or key=value overrides")
        loaded = OmegaConf.load(namespace.config)
        if not isinstance(loaded, DictConfig):
            raise ValueError("the top level of a config file must be a mapping")
        if "config" in loaded:
            raise ValueError("Cannot use 'config' within a config file")
        self.set_defaults(**OmegaConf.to_container(loaded, resolve=False))
        namespace, rest = super().parse_known_args(*args, **kwargs)
        del namespace.config
        return namespace, rest


def parse(recipe_main: Recipe) -> Callable[..., Any]:
    """Wrap ``recipe_main(cfg)`` so it reads ``--config file.yaml k=v ...`` from ``sys.argv``."""

    @functools.wraps(recipe_main)
    def wrapper(*args: Any, **kwargs: Any) -> Any:
        parser = TuneRecipeArgumentParser(
            description=recipe_main.__doc__, formatter_class=argparse.RawDescriptionHelpFormatter
        )
        yaml_args, cli_args = parser.parse_known_args()
        conf = _merge_yaml_and_cli_args(yaml_args, cli_args)
        sys.exit(recipe_main(conf))

    return wrapper
