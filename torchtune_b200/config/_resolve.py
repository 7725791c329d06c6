"""Dotted-path → Python object resolution with a compatibility alias.

YAML files written for the reference name components as ``torchtune.<path>``;
those paths are transparently mapped onto this package so such configs run
unmodified (parity: torchtune/config/_utils.py:37-118).
"""
from __future__ import annotations

import importlib
import inspect
from typing import Any, Dict, Optional

from ._errors import InstantiationError

_ALIASES = {"torchtune": "torchtune_b200"}

# Components of packages that are not part of this framework and have a built-in counterpart.  They are used only when the named
# package cannot be imported: with it installed, the config gets exactly what it names.
_STAND_INS = {
    "bitsandbytes.optim.PagedAdamW8bit": "torchtune_b200.optim.AdamW8bit",
    "bitsandbytes.optim.AdamW8bit": "torchtune_b200.optim.AdamW8bit",
    "bitsandbytes.optim.PagedAdamW": "torchtune_b200.optim.AdamW",
    "torchao.optim.AdamW8bit": "torchtune_b200.optim.AdamW8bit",
    "torchao.optim.AdamW4bit": "torchtune_b200.optim.AdamW8bit",
    "torchao.optim.AdamWFp8": "torchtune_b200.optim.AdamW8bit",
    "torchao.optim.CPUOffloadOptimizer": "torchtune_b200.optim.resident_optimizer",
}


def _alias(path: str) -> str:
    head, _, tail = path.partition(".")
    if head in _ALIASES:
        return _ALIASES[head] + ("." + tail if tail else "")
    return path


def has_component(node: Any) -> bool:
    from ._node import DictConfig

    return isinstance(node, (dict, DictConfig)) and "_component_" in node


def get_component_from_path(path: str, caller_globals: Optional[Dict[str, Any]] = None) -> Any:
    if not isinstance(path, str) or not path:
        raise InstantiationError(f"Invalid path: '{path}'")
    pieces = path.split(".")
    if "" in pieces:
        raise ValueError(f"Invalid dotstring. Relative imports are not supported. Got path={path!r}.")
    path = _alias(path)
    pieces = path.split(".")

    if len(pieces) == 1:
        try:
            return importlib.import_module(pieces[0])
        except ImportError:
            pass
        scope = caller_globals
        described = "the provided globals"
        if scope is None:
            described = "the caller's globals"
            frame = inspect.currentframe()
            scope = frame.f_back.f_globals if frame and frame.f_back else {}
        if pieces[0] in scope:
            return scope[pieces[0]]
        raise InstantiationError(
            f"Could not resolve '{pieces[0]}': not a module and not found in {described}."
        )

    module_name, attr = ".".join(pieces[:-1]), pieces[-1]
    try:
        module = importlib.import_module(module_name)
    except ImportError as exc:
        if path in _STAND_INS:
            import logging

            logging.getLogger(__name__).warning(f"{path} is not installed: using {_STAND_INS[path]} in its place")
            return get_component_from_path(_STAND_INS[path], caller_globals)
        # allow "pkg.module.Class.method"-style paths one level deep
        if len(pieces) > 2:
            try:
                owner = get_component_from_path(module_name, caller_globals)
                return getattr(owner, attr)
            except (InstantiationError, AttributeError):
                pass
        raise InstantiationError(f"Could not import module '{module_name}': {exc}.") from exc
    try:
        return getattr(module, attr)
    except AttributeError as exc:
        try:
            return importlib.import_module(path)
        except ImportError:
            raise InstantiationError(f"Module '{module_name}' has no attribute '{attr}'.") from exc
