"""Process-group plumbing used by the recipes
(parity: torchtune/training/_distributed.py:184-335, 486-611).

One process drives one GPU; ``torch.distributed`` (NCCL on CUDA, gloo on CPU) carries the
small control-plane collectives, while bulk gradient / parameter traffic goes through the
package's own peer-memory kernels (:mod:`torchtune_b200.parallel`).
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.mesh import ParallelDims  # re-exported
from ..utils import get_logger
from ..utils._device import get_world_size_and_rank

_log = get_logger()

VALID_BACKENDS_FOR_MEMORY_STATS = ("cuda",)


def is_distributed() -> bool:
    """True when the launcher exported a multi-process environment (RANK, WORLD_SIZE,
    MASTER_ADDR, MASTER_PORT) and ``torch.distributed`` is usable."""
    need = ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK")
    return dist.is_available() and all(os.environ.get(k) for k in need)


def get_distributed_backend(device_type: str, offload_ops_to_cpu: bool = False) -> str:
    """``nccl`` for CUDA, ``gloo`` for CPU.  With ``offload_ops_to_cpu`` a combined
    ``cuda:nccl,cpu:gloo`` backend is returned so CPU tensors (offloaded state dicts) can take
    part in collectives."""
    backend = {"cuda": "nccl", "cpu": "gloo"}.get(device_type)
    if backend is None:
        backend = dist.Backend.default_device_backend_map.get(device_type, "gloo")
    if offload_ops_to_cpu and device_type != "cpu":
        backend = f"{device_type}:{backend},cpu:gloo"
    return backend


def init_distributed(**kwargs: Any) -> bool:
    """Initialise the default process group when launched by a multi-process launcher.
    Returns whether a group was created."""
    if not is_distributed():
        return False
    if dist.is_initialized():
        raise RuntimeError("torch.distributed already initialized.")
    dist.init_process_group(**kwargs)
    return True


def set_torch_num_threads() -> None:
    """Split the host cores between the local ranks (intra-op CPU threads)."""
    local = int(os.environ.get("LOCAL_WORLD_SIZE", 1))
    n = max((os.cpu_count() or 1) // max(local, 1), 1)
    torch.set_num_threads(n)
    _log.info(f"Set intra op parallelism no. of threads to {n}")


def _broadcast_tensor(t: torch.Tensor, src: int = 0) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized():
        dev = t.device
        if dist.get_backend() == "nccl":
            t = t.to(torch.device("cuda", torch.cuda.current_device()))
        dist.broadcast(t, src=src)
        return t.to(dev)
    return t


def validate_no_params_on_meta_device(model: nn.Module) -> None:
    for name, t in list(model.named_parameters()) + list(model.named_buffers()):
        if t.is_meta:
            raise RuntimeError(f"Unexpected param or buffer {name} on meta device.")


def materialize(model: nn.Module, device: torch.device) -> nn.Module:
    """Give storage to a model built under ``torch.device('meta')`` and rebuild derived
    buffers (RoPE tables, KV caches keep their lazily-built state)."""
    if any(p.is_meta for p in model.parameters()) or any(b.is_meta for b in model.buffers()):
        model.to_empty(device=device)
        with device:
            for m in model.modules():
                if hasattr(m, "rope_init"):
                    m.rope_init()
                if hasattr(m, "initialize_parameters") and not isinstance(m, nn.modules.lazy.LazyModuleMixin):
                    m.initialize_parameters()
    return model


def load_from_full_model_state_dict(model: nn.Module, full_sd: Dict[str, Any], device: torch.device, strict: bool = False, cpu_offload: bool = False):
    """Load a full (unsharded, CPU) state dict into a resident model; every rank reads the
    same tensors, so no collective is needed.  NF4 base weights are quantised on the way in
    by the modules' own load hooks."""
    return model.load_state_dict(full_sd, strict=strict)


def gather_cpu_state_dict(model: nn.Module, is_rank_zero: bool, device: Optional[torch.device] = None, adapter_weights_only: bool = False) -> Dict[str, Any]:
    """Full state dict on the host of rank 0 (other ranks get ``{}``).  Parameters are
    resident on every rank, so this is a device→host copy, not a gather."""
    if not is_rank_zero:
        return {}
    sd = model.state_dict()
    if adapter_weights_only:
        from ..modules.peft import get_adapter_state_dict

        sd = get_adapter_state_dict(sd)
    return {k: v.detach().to("cpu") for k, v in sd.items()}


def get_full_optimizer_state_dict(model: nn.Module, opt, is_rank_zero: bool, device: Optional[torch.device] = None) -> Dict[str, Any]:
    """World-size independent optimizer state on rank 0 (see
    :meth:`torchtune_b200.parallel.ShardedAdamW.full_state_dict`)."""
    if hasattr(opt, "full_state_dict"):
        return opt.full_state_dict(is_rank_zero)
    return opt.state_dict() if is_rank_zero else {}


def load_from_full_optimizer_state_dict(model: nn.Module, opt, full_sd: Dict[str, Any], device: Optional[torch.device] = None) -> None:
    if hasattr(opt, "load_full_state_dict"):
        opt.load_full_state_dict(full_sd)
    else:
        opt.load_state_dict(full_sd)


__all__ = [
    "ParallelDims",
    "VALID_BACKENDS_FOR_MEMORY_STATS",
    "is_distributed",
    "get_distributed_backend",
    "init_distributed",
    "set_torch_num_threads",
    "get_world_size_and_rank",
    "validate_no_params_on_meta_device",
    "materialize",
    "load_from_full_model_state_dict",
    "gather_cpu_state_dict",
    "get_full_optimizer_state_dict",
    "load_from_full_optimizer_state_dict",
]
