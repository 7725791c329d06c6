"""YAML + command-line merging and config logging (parity: torchtune/config/_utils.py:18-231)."""
from __future__ import annotations

from argparse import Namespace
from typing import Any, Dict, List

from ._node import DictConfig, OmegaConf
from ._resolve import get_component_from_path as _get_component_from_path  # noqa: F401 (public alias)
from ._resolve import has_component as _has_component


def log_config(recipe_name: str, cfg: DictConfig) -> None:
    """Rank-0 dump of the resolved config, keys sorted."""
    from ..utils import get_logger, get_world_size_and_rank

    _, rank = get_world_size_and_rank()
    if rank != 0:
        return
    text = OmegaConf.to_yaml(cfg, resolve=True, sort_keys=True)
    get_logger("DEBUG").info(msg=f"Running {recipe_name} with resolved config:\n\n{text}")
    for key, why in REFERENCE_ONLY_KEYS.items():
        if key in cfg and cfg.get(key) not in (None, False):
            get_logger("DEBUG").info(msg=f"config key `{key}` is accepted for configs written for the reference and has no effect here: {why}")


# Top-level keys of the reference's recipes that steer machinery this framework does not have.  A config that sets one still runs.
REFERENCE_ONLY_KEYS: Dict[str, str] = {
    "fsdp_reshard_after_forward": "the sharded-parameter engine always frees a layer's gathered parameters after use (set `shard_parameters: False` for resident parameters)",
    "custom_sharded_layers": "every parameter is sharded bucket by bucket, no layer needs a sharding unit of its own",
    "fsdp_cpu_offload": "parameters, gradients and optimizer state stay in the 180 GB of device memory",
    "enable_expandable_segments": "the large buffers (flat parameter / gradient stores, peer buffers) are allocated once, outside the caching allocator",
    "low_cpu_ram": "checkpoints are memory-mapped and copied to the device tensor by tensor",
    "use_distributed_state_dict": "sharded models load from the full state dict layer by layer",
    "use_flex": "attention masks are structured descriptions lowered inside the attention kernel",
    "compile": "the hot path is hand-written kernels; there is no tracing compiler step",
}


def _remove_key_by_dotpath(tree: Dict[str, Any], dotpath: str) -> None:
    """Delete ``a.b.c`` from nested dicts, pruning parents that become empty.

    Component nodes can never be removed this way.
    """
    keys = dotpath.split(".")
    chain = [tree]
    for k in keys[:-1]:
        chain.append(chain[-1][k])

    def drop(container: Dict[str, Any], key: str) -> None:
        if _has_component(container[key]):
            raise ValueError(f"Removing components from CLI is not supported: ~{dotpath}")
        del container[key]

    drop(chain[-1], keys[-1])
    for depth in range(len(keys) - 2, -1, -1):
        if chain[depth + 1]:
            break
        drop(chain[depth], keys[depth])


def _merge_yaml_and_cli_args(yaml_args: Namespace, cli_args: List[str]) -> DictConfig:
    """Overlay ``key=value`` overrides on the YAML defaults.

    * ``key=dotted.path`` on a component node rewrites its ``_component_``.
    * ``~key`` deletes a (non-component) key.
    * the literal ``None`` becomes null; ``max_filename`` stays a string.
    """
    base: Dict[str, Any] = vars(yaml_args)
    overrides: List[str] = []
    for raw in cli_args:
        if raw.startswith("~"):
            dotpath = raw[1:].split("=")[0]
            if "_component_" in dotpath:
                raise ValueError(f"Removing components from CLI is not supported: ~{dotpath}")
            try:
                _remove_key_by_dotpath(base, dotpath)
            except (KeyError, TypeError):
                raise ValueError(f"Could not find key {dotpath} in yaml config to remove") from None
            except ValueError as exc:
                if "not supported" in str(exc):
                    raise ValueError(f"Could not find key {dotpath} in yaml config to remove") from None
                raise
            continue
        key, sep, value = raw.partition("=")
        if not sep or "=" in value and not (value.startswith(("'", '"', "[", "{"))):
            raise ValueError(f"Command-line overrides must be in the form of key=value, got {raw}")
        if key in base and _has_component(base[key]):
            key += "._component_"
        if value == "None":
            value = "null"
        if "max_filename" in key:
            value = f"'{value}'"
        overrides.append(f"{key}={value}")
    return OmegaConf.merge(OmegaConf.create(base), OmegaConf.from_dotlist(overrides))
