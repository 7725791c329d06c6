"""Memory-saving utilities (parity: torchtune/training/memory.py:26-294 and
torchtune/training/activations.py:19-88)."""
from __future__ import annotations

import gc
import logging
from typing import Any, Callable, Dict, Optional, Set, Type, Union

import torch
from torch import nn
from torch.optim.lr_scheduler import LRScheduler
from torch.utils.checkpoint import checkpoint

from ..utils import get_logger

_log = get_logger()

ACWrapPolicyType = Union[Set[Type], Callable[[nn.Module, bool, int], bool]]


class CheckpointedLayer(nn.Module):
    """Wraps a layer so its activations are recomputed in backward.  The wrapped module
    stays reachable under the *same* attribute path (no ``_checkpoint_wrapped_module``
    prefix in state-dict keys)."""

    def __init__(self, inner: nn.Module):
        super().__init__()
        self.__dict__["_inner_ref"] = inner
        self._modules = inner._modules
        self._parameters = inner._parameters
        self._buffers = inner._buffers
        self.inner_cls = type(inner)

    @property
    def inner(self) -> nn.Module:
        return self.__dict__["_inner_ref"]

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.__dict__["_inner_ref"], name)

    def forward(self, *args, **kwargs):
        if not torch.is_grad_enabled():
            return self.inner(*args, **kwargs)
        return checkpoint(self.inner, *args, use_reentrant=False, preserve_rng_state=True, **kwargs)


def _swap_children(model: nn.Module, predicate: Callable[[nn.Module], bool]) -> int:
    count = 0
    for parent in list(model.modules()):
        if isinstance(parent, CheckpointedLayer):
            continue
        for name, child in list(parent._modules.items()):
            if child is not None and not isinstance(child, CheckpointedLayer) and predicate(child):
                parent._modules[name] = CheckpointedLayer(child)
                count += 1
    return count


def set_activation_checkpointing(model: nn.Module, auto_wrap_policy: ACWrapPolicyType, **kwargs) -> None:
    """Recompute-in-backward for every sub-module selected by ``auto_wrap_policy`` (a set
    of module classes or a ``(module, recurse, nonwrapped_numel) -> bool`` callable)."""
    if isinstance(auto_wrap_policy, (set, frozenset, list, tuple)):
        classes = tuple(auto_wrap_policy)
        _swap_children(model, lambda m: isinstance(m, classes))
    else:
        _swap_children(model, lambda m: bool(auto_wrap_policy(m, False, 0)))


def apply_selective_activation_checkpointing(model: nn.Module, ac_mode: str, ac_option: Optional[Union[int, str]]) -> None:
    """``ac_mode='full'`` checkpoints every decoder layer; ``'selective'`` with an integer
    ``ac_option=k`` checkpoints every k-th layer (k=1 all, 2 every other, …)."""
    from ..modules import TransformerCrossAttentionLayer, TransformerSelfAttentionLayer

    layer_types = (TransformerSelfAttentionLayer, TransformerCrossAttentionLayer)
    if ac_mode not in ("full", "selective"):
        raise ValueError(f"Invalid AC mode: {ac_mode}. Valid modes: full, selective")
    if ac_mode == "full":
        set_activation_checkpointing(model, set(layer_types))
        return
    try:
        every = int(ac_option)
    except (TypeError, ValueError):
        raise ValueError(f"Invalid selective AC option: {ac_option}. Valid options: an integer layer frequency") from None
    if every <= 0:
        raise ValueError(f"Selective layer AC expects a positive int as selective_ac_option but got {every}")
    counter = {"n": 0}

    def pick(m: nn.Module) -> bool:
        if not isinstance(m, layer_types):
            return False
        counter["n"] += 1
        return every == 1 or counter["n"] % every == 0

    _swap_children(model, pick)


def cleanup_before_training() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()


class OptimizerInBackwardWrapper:
    """State-dict / LR facade over a ``{param_name: optimizer}`` map used when optimizer
    steps run inside backward."""

    def __init__(self, optim_map: Dict[str, torch.optim.Optimizer]):
        self.optim_map = optim_map
        self.lr_scheduler: Optional[LRScheduler] = None

    def state_dict(self) -> Dict[str, Any]:
        return {name: opt.state_dict() for name, opt in self.optim_map.items()}

    def load_state_dict(self, optim_ckpt_map: Dict[str, Any]) -> None:
        seen = set()
        for name, sd in optim_ckpt_map.items():
            if name not in self.optim_map:
                raise RuntimeError(f"Trying to load optimizer state for unexpected param {name}")
            self.optim_map[name].load_state_dict(sd)
            seen.add(name)
        missing = set(self.optim_map) - seen
        if missing:
            raise RuntimeError(f"Expected to load optimizer state for params {missing}!")

    def get_optim_key(self, key: str) -> Any:
        return next(iter(self.optim_map.values())).param_groups[0][key]

    def set_lr_scheduler(self, lr_scheduler: LRScheduler) -> None:
        """Mirror one scheduler's learning rate onto every per-parameter optimizer."""
        self.lr_scheduler = lr_scheduler
        original_step = lr_scheduler.step

        def step_and_sync(*args, **kwargs):
            original_step(*args, **kwargs)
            lr = lr_scheduler.get_last_lr()[0]
            for opt in self.optim_map.values():
                for g in opt.param_groups:
                    g["lr"] = lr

        lr_scheduler.step = step_and_sync

    def step_lr_scheduler(self, epoch: Optional[int] = None) -> None:
        if self.lr_scheduler is None:
            raise RuntimeError("LR scheduler is not set")
        self.lr_scheduler.step(epoch)

    def get_last_lr(self) -> float:
        if self.lr_scheduler is None:
            raise RuntimeError("LR scheduler is not set")
        return self.lr_scheduler.get_last_lr()[0]


def create_optim_in_bwd_wrapper(model: nn.Module, optim_dict: Dict[torch.nn.Parameter, torch.optim.Optimizer]) -> OptimizerInBackwardWrapper:
    return OptimizerInBackwardWrapper({n: optim_dict[p] for n, p in model.named_parameters() if p in optim_dict})


def register_optim_in_bwd_hooks(model: nn.Module, optim_dict: Dict[torch.nn.Parameter, torch.optim.Optimizer]) -> None:
    """Step + zero each parameter's optimizer as soon as its gradient is accumulated."""

    def fire(param) -> None:
        optim_dict[param].step()
        optim_dict[param].zero_grad()

    for p in model.parameters():
        if p.requires_grad:
            p.register_post_accumulate_grad_hook(fire)


def get_memory_stats(device: torch.device, reset_stats: bool = True) -> Dict[str, float]:
    """Peak active / allocated / reserved memory in GiB since the last reset."""
    if device.type != "cuda":
        raise ValueError(f"Logging memory stats is only supported on CUDA devices, got {device}")
    gib = 1024**3
    stats = {
        "peak_memory_active": torch.cuda.memory_stats(device).get("active_bytes.all.peak", 0) / gib,
        "peak_memory_alloc": torch.cuda.max_memory_allocated(device) / gib,
        "peak_memory_reserved": torch.cuda.max_memory_reserved(device) / gib,
    }
    if reset_stats:
        torch.cuda.reset_peak_memory_stats(device)
    return stats


def log_memory_stats(stats: Dict[str, float], message: str = "Memory stats after model init:") -> None:
    _log.info(
        f"{message}"
        f"\n\tGPU peak memory active: {stats['peak_memory_active']:.2f} GiB"
        f"\n\tGPU peak memory allocation: {stats['peak_memory_alloc']:.2f} GiB"
        f"\n\tGPU peak memory reserved: {stats['peak_memory_reserved']:.2f} GiB"
    )
