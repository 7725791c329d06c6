"""Recursive ``_component_`` instantiation (parity: torchtune/config/_instantiate.py:27-167)."""
from __future__ import annotations

import copy
import inspect
import os
import sys
from typing import Any, Dict, Optional, Union

from ._errors import InstantiationError
from ._node import DictConfig, ListConfig, OmegaConf
from ._resolve import get_component_from_path


def _build(node: Any, positional: tuple, scope: Optional[Dict[str, Any]]) -> Any:
    if isinstance(node, dict):
        if "_component_" in node:
            target = get_component_from_path(node["_component_"], caller_globals=scope)
            kwargs = {k: _build(v, (), scope) for k, v in node.items() if k != "_component_"}
            return target(*positional, **kwargs)
        return {k: _build(v, (), scope) for k, v in node.items()}
    if isinstance(node, list):
        return [_build(v, (), scope) for v in node]
    return node


def instantiate(
    config: Union[Dict[str, Any], DictConfig, None],
    *args: Any,
    caller_globals: Optional[Dict[str, Any]] = None,
    **kwargs: Any,
) -> Any:
    """Create the object described by ``config``.

    ``config`` must hold a ``_component_`` dotted path; remaining keys become
    keyword arguments, nested component nodes are instantiated first.
    ``*args`` are passed positionally to the top-level component only and
    ``**kwargs`` override keys of the config.  Bare names (no dot) fall back to
    the caller's module globals.
    """
    if config is None:
        return None
    if isinstance(config, dict):
        config = OmegaConf.create(config)
    elif not isinstance(config, DictConfig):
        raise ValueError(f"instantiate only supports DictConfigs or dicts, got {type(config)}")
    if "_component_" not in config:
        raise InstantiationError(
            "Cannot instantiate specified object."
            "\nMake sure you've specified a _component_ field with a valid dotpath."
            f"\nGot config={config!r}."
        )
    if os.getcwd() not in sys.path:
        sys.path.append(os.getcwd())

    # Resolve against the original tree (interpolations may point outside this node).
    resolved = OmegaConf.to_container(config, resolve=True)
    objects = {}
    for key, value in kwargs.items():
        if isinstance(value, (DictConfig, ListConfig)):
            resolved[key] = OmegaConf.to_container(value, resolve=True)
        elif isinstance(value, (dict, list, str, int, float, bool)) or value is None:
            resolved[key] = copy.deepcopy(value)
        else:
            objects[key] = value  # live objects bypass recursion
            resolved.pop(key, None)

    if caller_globals is None:
        frame = inspect.currentframe()
        if frame is not None and frame.f_back is not None:
            caller_globals = frame.f_back.f_globals

    target = get_component_from_path(resolved["_component_"], caller_globals=caller_globals)
    built = {k: _build(v, (), caller_globals) for k, v in resolved.items() if k != "_component_"}
    built.update(objects)
    return target(*args, **built)
