"""Process-group plumbing used by the recipes
(parity: torchtune/training/_distributed.py:184-335, 486-611).

One process drives one GPU; ``torch.distributed`` (NCCL on CUDA, gloo on CPU) carries the
small control-plane collectives, while bulk gradient / parameter traffic goes through the
package's own peer-memory kernels (:mod:`torchtune_b200.parallel`).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

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
        # only what has no storage yet: tensors that already live somewhere (shards placed in a peer-visible store, parts of a
        # 4-bit base) keep their storage and their values
        for module in model.modules():
            for name, p in list(module._parameters.items()):
                if p is not None and p.is_meta:
                    module._parameters[name] = torch.nn.Parameter(torch.empty_like(p, device=device), requires_grad=p.requires_grad)
            for name, b in list(module._buffers.items()):
                if b is not None and b.is_meta:
                    module._buffers[name] = torch.empty_like(b, device=device)
        with device:
            for m in model.modules():
                if hasattr(m, "rope_init"):
                    m.rope_init()
                if hasattr(m, "initialize_parameters") and not isinstance(m, nn.modules.lazy.LazyModuleMixin):
                    m.initialize_parameters()
    return model


class LayerwisePreparer:
    """Gives storage and values to one sub-module at a time of a model built under ``torch.device('meta')``.

    The tensor- and expert-parallel conversions call it with every decoder layer right before they slice that layer
    (``prepare(module, "layers.3.")``) and once more for what is not a layer, so a model far larger than one GPU (70B dense,
    109B mixture of experts) never exists in full: at most one unsharded layer is alive next to the shards.  Values come
    from a full checkpoint state dict (``state_dict``; keys are model-level names) or, without one, from
    ``normal(0, init_std)`` drawn from a generator seeded by ``seed`` and the module's name — identical on every rank, so the
    ranks' shards are slices of the same matrices."""

    def __init__(self, device: torch.device, state_dict: Optional[Dict[str, Any]] = None, init_std: float = 0.02, seed: int = 1234):
        self.device, self.state_dict, self.init_std, self.seed = device, state_dict, init_std, seed

    def __call__(self, module: nn.Module, prefix: str = "") -> nn.Module:
        if any(t.is_meta for t in list(module.parameters()) + list(module.buffers())):
            module.to_empty(device=self.device)
            with self.device:
                for m in module.modules():
                    if hasattr(m, "rope_init"):
                        m.rope_init()
        if self.state_dict is not None:
            own = {k[len(prefix):]: v for k, v in self.state_dict.items() if k.startswith(prefix)} if prefix else {
                k: v for k, v in self.state_dict.items() if k in module.state_dict()}
            module.load_state_dict(own, strict=bool(prefix))
            return module
        import zlib

        gen = torch.Generator(device=self.device).manual_seed(self.seed + zlib.crc32(prefix.encode()))
        with torch.no_grad():
            for name, p in module.named_parameters():
                if p.dim() > 1:
                    p.normal_(0.0, self.init_std, generator=gen)
                elif "scale" in name or "norm" in name:
                    p.fill_(1.0)
                else:
                    p.zero_()
        return module


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


# ------------------------------------------------------------------------------ sharding / parallel helpers (recipe-facing names)
def get_shard_conditions(name: str, module: nn.Module, names_to_match: Optional[List[str]] = None, *args: Any, **kwargs: Any) -> bool:
    """``True`` for the modules that form their own shard unit: every decoder layer (a module path ending in ``layers.<int>``)
    and anything listed in ``names_to_match`` (torchtune/training/_distributed.py:612-658)."""
    if names_to_match and name in names_to_match:
        return True
    parts = name.split(".")
    return len(parts) >= 2 and parts[-2] == "layers" and parts[-1].isdigit()


def shard_model(model: nn.Module, shard_conditions=None, *, cpu_offload: bool = False, reshard_after_forward: bool = True, dp_mesh=None,
                device: Optional[torch.device] = None, min_numel: int = 1 << 16) -> nn.Module:
    """Shard the parameters of ``model`` over the data-parallel ranks (the call the reference's recipes make,
    torchtune/training/_distributed.py:661-714).  Here that means: the rows of every linear weight are split over the ranks in
    one peer-visible store and gathered inside the consuming GEMM (:func:`torchtune_b200.parallel.fsdp.shard_linear_weights`).
    ``shard_conditions`` / ``reshard_after_forward`` are accepted for signature parity: weights are always re-gathered per use,
    and the unit of sharding is the linear layer.  ``dp_mesh`` may be a process group (or ``None`` for all ranks)."""
    from ..parallel.fsdp import shard_linear_weights

    if cpu_offload:
        raise NotImplementedError("cpu_offload is not supported: 180 GB of device memory hold the sharded state")
    if device is None:
        first = next(model.parameters())
        device = first.device
    return shard_linear_weights(model, device, dp_mesh, min_numel=min_numel)


def prepare_mha_for_tp(model: nn.Module, tp_mesh) -> nn.Module:
    """Divide the head counts and width of every attention module by the tensor-parallel size so that reshapes inside
    attention see local shapes (torchtune/training/_distributed.py:717-778).  ``tp_mesh``: an int, a process group or anything
    with ``size()``.  (:func:`torchtune_b200.parallel.tp_model.tensor_parallelize` builds its own local attention modules and does
    not need this; it is kept for code that shards projections by hand.)"""
    from ..modules import MultiHeadAttention

    if isinstance(tp_mesh, int):
        size = tp_mesh
    elif hasattr(tp_mesh, "size") and callable(tp_mesh.size):
        size = tp_mesh.size()
    else:
        size = dist.get_world_size(tp_mesh)
    for m in model.modules():
        if isinstance(m, MultiHeadAttention):
            if m.num_heads % size or m.num_kv_heads % size or m.embed_dim % size:
                raise ValueError(f"tensor parallel size {size} must divide num_heads ({m.num_heads}), num_kv_heads ({m.num_kv_heads}) and embed_dim ({m.embed_dim})")
            m.num_heads //= size
            m.num_kv_heads //= size
            m.embed_dim //= size
    return model


def get_context_parallel_manager(*, enabled: bool = False, world_mesh=None, model: Optional[nn.Module] = None, cp=None):
    """Returns ``manager(buffers)``, a context manager that — when enabled — swaps every tensor in ``buffers`` for this rank's
    slice of its sequence dimension (dim 1) for the duration of the block and restores it afterwards
    (torchtune/training/_distributed.py:781-886).  ``cp``: a :class:`torchtune_b200.parallel.cp.ContextParallelContext` (the
    model must have been prepared with :func:`torchtune_b200.parallel.cp.context_parallelize`); ``world_mesh`` is accepted for
    signature parity."""
    import contextlib

    @contextlib.contextmanager
    def manager(buffers: Optional[List[torch.Tensor]] = None):
        if not enabled or cp is None or not buffers:
            yield
            return
        saved = []
        for t in buffers:
            keep = torch.empty(0, dtype=t.dtype, device=t.device).set_(t)
            saved.append(keep)
            t.set_(cp.shard_seq(keep, dim=1).contiguous())
        try:
            yield
        finally:
            for t, keep in zip(buffers, saved):
                t.set_(keep)

    return manager


def get_train_context(enable_loss_parallel: bool = False):
    """Returns a factory of context managers for one training step (torchtune/training/_distributed.py:889-902).  Under tensor
    parallelism the loss already runs on each rank's own token rows with the whole vocabulary, so there is nothing to switch on."""
    import contextlib

    def context():
        return contextlib.nullcontext()

    return context
