"""Config → parallel strategy for the distributed recipes.

The reference wires FSDP2 + DTensor TP/CP from the recipe config
(recipes/full_finetune_distributed.py:142-175, 586-686).  On 180 GB parts the default
here is *resident* data parallelism: full bf16 parameters on every rank in a flat
peer-visible buffer, sharded optimizer state, one fused reduce→AdamW→broadcast kernel per
step (:mod:`.dp`).  The recipe-facing surface is the one :class:`engine.sft.SFTTrainer`
drives: ``shard_model``, ``build_optimizer``, ``optimizer_step``, state-dict gathers and the
small collectives.
"""
from __future__ import annotations

import datetime
import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..utils import get_logger
from .dp import DataParallelEngine, ShardedAdamW
from .mesh import ParallelDims

_log = get_logger()

_FUSED_ADAMW = {"torch.optim.AdamW", "torchtune_b200.optim.AdamW", "torchtune_b200.optim.adamw.AdamW", "torchao.optim.AdamW8bit", "bitsandbytes.optim.PagedAdamW8bit", "bitsandbytes.optim.PagedAdamW"}


class ReplicatedOptimizer:
    """Any ``torch.optim`` optimizer under data parallelism: the flat gradient buffer is summed
    across ranks with one all-reduce, scaled/clipped, and every rank applies the same update."""

    def __init__(self, engine: "ParallelStrategy", optimizer: torch.optim.Optimizer):
        self.engine, self.optimizer = engine, optimizer
        self.last_grad_norm: Optional[torch.Tensor] = None

    torch_optimizer = property(lambda self: self.optimizer)
    param_groups = property(lambda self: self.optimizer.param_groups)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.flat.reset_grad_flags()
        for p in self.engine.flat.params:
            p.grad = None

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd) -> None:
        self.optimizer.load_state_dict(sd)

    def full_state_dict(self, is_rank_zero: bool = True, group=None):
        return self.optimizer.state_dict() if is_rank_zero else {}

    def load_full_state_dict(self, sd) -> None:
        self.optimizer.load_state_dict(sd)

    def step(self, grad_scale=1.0, max_grad_norm: Optional[float] = None, group=None) -> None:
        flat = self.engine.flat
        g = flat.flat_grad
        if self.engine.world > 1:
            if g.dtype == torch.bfloat16 and g.device.type == "cpu":
                g32 = g.float()
                dist.all_reduce(g32, group=group)
                g.copy_(g32)
            else:
                dist.all_reduce(g, group=group)
        g.mul_(grad_scale if not isinstance(grad_scale, torch.Tensor) else grad_scale.to(g.dtype))
        self.last_grad_norm = None
        if max_grad_norm is not None:
            norm = g.float().norm()
            self.last_grad_norm = norm
            g.mul_(torch.clamp(float(max_grad_norm) / (norm + 1e-6), max=1.0).to(g.dtype))
        for p in flat.params:
            p.grad = p._grad_buffer
        self.optimizer.step()
        for p in flat.params:
            p.grad = None


class ParallelStrategy(DataParallelEngine):
    """Process group + parallel dims + resident data-parallel engine, built from recipe config keys
    ``tensor_parallel_dim``, ``context_parallel_dim``, ``data_parallel_shard_dim``,
    ``data_parallel_replicate_dim`` (same names as the reference's distributed recipes)."""

    def __init__(self, cfg, device: torch.device):
        if not dist.is_initialized():
            backend = "nccl" if device.type == "cuda" else "gloo"
            kwargs: Dict[str, Any] = {"backend": backend}
            if device.type == "cuda":
                kwargs["device_id"] = device
            timeout_s = cfg.get("process_group_timeout_s") if hasattr(cfg, "get") else None
            if timeout_s:
                kwargs["timeout"] = datetime.timedelta(seconds=float(timeout_s))
            if all(os.environ.get(k) for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")):
                dist.init_process_group(**kwargs)
                self._owns_group = True
            else:
                self._owns_group = False
        else:
            self._owns_group = False
        world = dist.get_world_size() if dist.is_initialized() else 1
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
        self.dims = ParallelDims(
            dp_replicate=get("data_parallel_replicate_dim", 1) or 1,
            dp_shard=get("data_parallel_shard_dim", -1) or -1,
            tp=get("tensor_parallel_dim", 1) or 1,
            cp=get("context_parallel_dim", 1) or 1,
            world_size=world,
        )
        if self.dims.tp_enabled or self.dims.cp_enabled:
            raise NotImplementedError(
                "tensor_parallel_dim / context_parallel_dim > 1 are not wired into the recipes yet; "
                "an 8-way data-parallel job holds models up to ~70B parameters resident on 180 GB GPUs"
            )
        super().__init__(device=device, group=None)
        self._cpu_offload = bool(get("fsdp_cpu_offload", False))

    # sizes -------------------------------------------------------------------------------
    @property
    def non_data_parallel_size(self) -> int:  # type: ignore[override]
        return self.dims.non_data_parallel_size

    @property
    def min_seq_len_divisor(self) -> int:  # type: ignore[override]
        return self.dims.min_seq_len_divisor

    # model -------------------------------------------------------------------------------
    def shard_model(self, model: nn.Module, cfg, base_sd: Dict[str, Any], adapter_sd: Optional[Dict[str, Any]] = None, *, dtype: torch.dtype = torch.bfloat16, strict: bool = True) -> nn.Module:
        from ..training._distributed import materialize, validate_no_params_on_meta_device

        materialize(model, self.device)
        is_lora = not strict
        if is_lora:
            from ..modules.peft import validate_missing_and_unexpected_for_lora

            base_missing, base_unexpected = model.load_state_dict(base_sd, strict=False)
            lora_missing = lora_unexpected = None
            if adapter_sd is not None:
                lora_missing, lora_unexpected = model.load_state_dict(adapter_sd, strict=False)
            validate_missing_and_unexpected_for_lora(
                state_dict_keys=list(model.state_dict().keys()), base_missing=base_missing, base_unexpected=base_unexpected, lora_missing=lora_missing, lora_unexpected=lora_unexpected
            )
            if adapter_sd is None:
                for m in model.modules():
                    if hasattr(m, "initialize_dora_magnitude"):
                        m.initialize_dora_magnitude()
        else:
            model.load_state_dict(base_sd, strict=True)
        validate_no_params_on_meta_device(model)
        self.prepare(model)
        if self.world > 1:
            # adapters are initialised with rank-dependent seeds: rank 0's values win
            flat = self.flat.flat_param
            if flat.device.type == "cpu" and flat.dtype == torch.bfloat16:
                tmp = flat.float()
                dist.broadcast(tmp, src=0)
                flat.copy_(tmp)
            else:
                dist.broadcast(flat, src=0)
        return model

    # optimizer ---------------------------------------------------------------------------
    def build_optimizer(self, model: nn.Module, cfg_optimizer=None, opt_state: Optional[Dict[str, Any]] = None, **kwargs: Any):
        if self.flat is None:
            raise RuntimeError("shard_model(model, …) must run before build_optimizer")
        if cfg_optimizer is None or not hasattr(cfg_optimizer, "get"):
            if isinstance(cfg_optimizer, (int, float)):
                kwargs.setdefault("lr", float(cfg_optimizer))
            opt = DataParallelEngine.build_optimizer(self, model, **kwargs)
        else:
            from .. import config

            target = cfg_optimizer.get("_component_", "torch.optim.AdamW")
            target = target.replace("torchtune.", "torchtune_b200.", 1) if target.startswith("torchtune.") else target
            params = {k: v for k, v in cfg_optimizer.items() if k != "_component_"}
            if target in _FUSED_ADAMW and not params.get("amsgrad", False) and not params.get("maximize", False):
                opt = ShardedAdamW(
                    self.flat,
                    self.rank,
                    self.world,
                    lr=float(params.get("lr", 1e-3)),
                    betas=tuple(params.get("betas", (0.9, 0.999))),
                    eps=float(params.get("eps", 1e-8)),
                    weight_decay=float(params.get("weight_decay", 1e-2)),
                )
            else:
                opt = ReplicatedOptimizer(self, config.instantiate(cfg_optimizer, self.flat.params))
        if opt_state:
            opt.load_full_state_dict(opt_state)
        return opt

    def optimizer_step(self, model: nn.Module, optimizer, grad_scale, clip_grad_norm: Optional[float] = None):
        clip = float(clip_grad_norm) if clip_grad_norm is not None else None
        return super().optimizer_step(model, optimizer, grad_scale, clip)

    # state dicts -------------------------------------------------------------------------
    def gather_full_state_dict(self, model: nn.Module) -> Dict[str, Any]:
        from ..training._distributed import gather_cpu_state_dict

        return gather_cpu_state_dict(model, self.rank == 0, self.device)

    def gather_optimizer_state_dict(self, model: nn.Module, optimizer) -> Dict[str, Any]:
        return optimizer.full_state_dict(self.rank == 0, group=self.group)

    def shutdown(self) -> None:
        super().shutdown()
        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()


def init_from_config(cfg, device: torch.device) -> ParallelStrategy:
    return ParallelStrategy(cfg, device)
