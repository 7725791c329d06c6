"""Signature check of every top-level component (parity: torchtune/config/_validate.py:14-45)."""
from __future__ import annotations

import inspect

from ._errors import ConfigError
from ._node import DictConfig, OmegaConf
from ._resolve import get_component_from_path, has_component


def validate(cfg: DictConfig) -> None:
    """Bind each top-level component's kwargs to its signature.

    A component whose only problem is a missing *required* argument is accepted
    (recipes supply those positionally, e.g. the tokenizer for a dataset).
    All other mismatches are collected and raised together as ``ConfigError``.
    """
    problems = []
    for key, node in cfg.items():
        if not has_component(node):
            continue
        try:
            target = get_component_from_path(node.get("_component_"))
            kwargs = {k: v for k, v in OmegaConf.to_container(node, resolve=False).items() if k != "_component_"}
            sig = inspect.signature(target)
            try:
                sig.bind(**kwargs)
            except TypeError as exc:
                if "missing a required argument" in str(exc):
                    sig.bind_partial(**kwargs)
                else:
                    raise
        except TypeError as exc:
            problems.append(TypeError(f"{key}: {exc}"))
    if problems:
        raise ConfigError(problems)
