"""Adapter bookkeeping helpers (parity: torchtune/modules/peft/_utils.py:17-417)."""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Generator, Iterable, List, Literal, Optional, Protocol, Set, Union, runtime_checkable

import torch
import torch.distributed as dist
from torch import nn

LORA_ATTN_MODULES = Literal["q_proj", "k_proj", "v_proj", "output_proj"]
_EXPERT_SUFFIXES = tuple(f".lora_{p}_{ab}" for p in ("gate", "down", "up") for ab in ("a", "b"))
_LINEAR_SUFFIXES = (".lora_a.weight", ".lora_b.weight", ".magnitude")


@runtime_checkable
class AdapterModule(Protocol):
    """Any module that lists its adapter parameter names via ``adapter_params()``."""

    def adapter_params(self) -> List[str]:
        ...


def _is_adapter_module(m: nn.Module) -> bool:
    return callable(getattr(m, "adapter_params", None))


def _is_adapter_key(key: str) -> bool:
    return "lora" in key or "magnitude" in key


def get_adapter_params(model: nn.Module) -> Dict[str, nn.Parameter]:
    """Fully-qualified name → parameter for every adapter parameter in ``model``."""
    found: Dict[str, nn.Parameter] = {}
    for mod_name, mod in model.named_modules():
        if not _is_adapter_module(mod):
            continue
        wanted = list(mod.adapter_params())
        for p_name, p in mod.named_parameters(recurse=True):
            if p_name in wanted:
                found[f"{mod_name}.{p_name}" if mod_name else p_name] = p
                wanted.remove(p_name)
        assert not wanted, f"Adapter params {wanted} not converted"
    return found


def set_trainable_params(model: nn.Module, adapter_params: Union[Dict[str, Any], Set[str]]) -> None:
    """Freeze everything except the named adapter parameters."""
    for name, p in model.named_parameters():
        p.requires_grad_(name in adapter_params)


def get_lora_module_names(lora_attn_modules: List[str], apply_lora_to_mlp: bool, apply_lora_to_output: bool) -> List[str]:
    names = list(lora_attn_modules)
    if apply_lora_to_mlp:
        names += ["w1", "w2", "w3"]
    if apply_lora_to_output:
        names.append("output")
    return names


def get_adapter_state_dict(state_dict: Dict[str, Any], device: Optional[str] = "cpu") -> Dict[str, Any]:
    """Adapter-only subset of an unsharded state dict, moved to ``device``."""
    return {k: v.to(device) for k, v in state_dict.items() if _is_adapter_key(k)}


def _strip_any(key: str, suffixes: Iterable[str]) -> str:
    for s in suffixes:
        if key.endswith(s):
            return key[: -len(s)]
    return key


def _get_lora_modules(state_dict: Dict[str, Any]) -> Set[str]:
    return {_strip_any(k, _LINEAR_SUFFIXES) for k in state_dict if _is_adapter_key(k) and "experts" not in k}


def _get_lora_moe_modules(state_dict: Dict[str, Any]) -> Set[str]:
    return {_strip_any(k, _EXPERT_SUFFIXES) for k in state_dict if "lora" in k and "experts" in k}


@torch.no_grad()
def get_merged_lora_ckpt(state_dict: Dict[str, Any], rank: int, alpha: float, use_distributed_barriers: bool = False) -> Dict[str, Any]:
    """Fold every adapter into its base weight **in place** and drop the adapter keys.

    * LoRA:   ``W += (alpha/rank) · B A``
    * DoRA:   ``W = m / ||W + ΔW||_row · (W + ΔW)``
    * expert: ``W_e += (alpha/rank) · A_e B_e`` for the ``[E, in, out]`` layout
    """
    s = alpha / rank

    def sync() -> None:
        if use_distributed_barriers:
            dist.barrier()

    for mod in sorted(_get_lora_modules(state_dict) | _get_lora_moe_modules(state_dict)):
        if "experts" in mod:
            for proj in ("gate", "up", "down"):
                a = state_dict.pop(f"{mod}.lora_{proj}_a")  # [E, in, r]
                b = state_dict.pop(f"{mod}.lora_{proj}_b")  # [E, r, out]
                sync()
                state_dict[f"{mod}.{proj}_proj"] += s * torch.bmm(a, b)
            continue
        a = state_dict.pop(f"{mod}.lora_a.weight")
        b = state_dict.pop(f"{mod}.lora_b.weight")
        mag = state_dict.pop(f"{mod}.magnitude", None)
        sync()
        delta = s * (b @ a)
        if mag is None:
            state_dict[f"{mod}.weight"] += delta
        else:
            merged = state_dict[f"{mod}.weight"].to(a.dtype) + delta
            sync()
            merged *= (mag / torch.linalg.norm(merged, dim=1)).view(-1, 1)
            state_dict[f"{mod}.weight"] = merged
    return state_dict


@contextlib.contextmanager
def disable_adapter(model: nn.Module) -> Generator[None, None, None]:
    """Run the body with every adapter switched off (base model behaviour)."""
    touched = [m for m in model.modules() if _is_adapter_module(m) and hasattr(m, "disabled")]
    for m in touched:
        m.disabled = True
    try:
        yield
    finally:
        for m in touched:
            m.disabled = False


def validate_missing_and_unexpected_for_lora(
    lora_attn_modules: Optional[List[str]] = None,
    apply_lora_to_mlp: Optional[bool] = None,
    apply_lora_to_output: Optional[bool] = None,
    state_dict_keys: Optional[List[str]] = None,
    base_missing: Optional[List[str]] = None,
    base_unexpected: Optional[List[str]] = None,
    lora_missing: Optional[List[str]] = None,
    lora_unexpected: Optional[List[str]] = None,
) -> None:
    """Check the results of two ``load_state_dict(strict=False)`` calls (base weights, then
    adapter weights): every base key must have come from the base load, every adapter key
    from the adapter load, and nothing unexpected may appear."""
    base_missing, lora_missing = list(base_missing or []), list(lora_missing or [])
    if state_dict_keys is not None:
        base_keys = {k for k in state_dict_keys if not _is_adapter_key(k)}
        lora_keys = {k for k in state_dict_keys if _is_adapter_key(k)}
        bm, lm = set(base_missing), set(lora_missing)
        problems = []
        for key in sorted((bm & lm) | (lm & lora_keys) | (bm & base_keys)):
            if key in base_keys:
                problems.append(f"- Missing non-LoRA key {key} from base model dict")
            elif key in lora_keys:
                problems.append(f"- Missing LoRA key {key} from adapter state dict")
            else:
                raise RuntimeError(f"Unexpected key found missing: {key}")
        if problems:
            raise RuntimeError("Missing keys when validating state dict: \n" + "\n".join(problems))
    else:
        assert lora_attn_modules is not None and apply_lora_to_mlp is not None and apply_lora_to_output is not None
        mods = get_lora_module_names(lora_attn_modules, apply_lora_to_mlp, apply_lora_to_output)

        def is_lora_param(k: str) -> bool:
            return any(f"{m}.lora" in k or f"{m}.magnitude" in k for m in mods)

        for k in base_missing:
            if not is_lora_param(k):
                raise RuntimeError(f"Missing non-LoRA key {k} from base model dict")
        for k in lora_missing:
            if is_lora_param(k):
                raise RuntimeError(f"Missing LoRA key {k} from adapter state dict")
    if base_unexpected:
        raise RuntimeError("Unexpected key loading base model")
    if lora_unexpected:
        raise RuntimeError("Unexpected key loading adapter")
