"""Several flat parameter stores behind one optimizer: the fused sharded AdamW for tensor- and expert-parallel models.

A tensor- or expert-parallel model has two kinds of parameters.  *Local* ones (projection shards, this rank's experts)
exist once per model replica, so their gradients are summed over the ranks that hold the same shard (the data-parallel
replica group; a single rank when there is one replica).  *Replicated* ones (embeddings, output head, norm scales, router,
shared expert, attention under expert parallelism) exist on every rank and every rank contributes a partial gradient
(its own tokens), so they are summed over the whole job.  Each kind gets its own :class:`~.dp.FlatParameters` store
over its own group, and the fused pull-reduce → AdamW → push kernel (``ops/csrc/comm.cu``) runs per store: the AdamW
moments of the replicated parameters are sharded over *all* ranks, those of a local shard over its replicas, and one
all-reduce of a scalar gives the global clipping norm (every element of every store is owned by exactly one rank).

The reference reaches the same state by composing FSDP2 over the data-parallel mesh with DTensor tensor parallelism
(recipes/full_finetune_distributed.py:630-692) and stepping ``torch.optim.AdamW`` on the DTensor shards.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from .dp import FlatParameters, ShardedAdamW
from .fabric import SOLO


class StoreSpec:
    """``params``: named parameters of one store; ``group``: the process group their gradients are summed over (``None`` =
    every rank, :data:`~.fabric.SOLO` = this rank alone)."""

    def __init__(self, name: str, params: Sequence[Tuple[str, nn.Parameter]], group: Any = None):
        self.name, self.params, self.group = name, list(params), group

    def size(self) -> Tuple[int, int]:
        if self.group is SOLO or not dist.is_initialized():
            return 1, 0
        return dist.get_world_size(self.group), dist.get_rank(self.group)


class MultiStoreAdamW:
    """AdamW over several :class:`FlatParameters` stores (one fused kernel per bucket and store).

    The ``torch.optim``-like surface (``param_groups``, ``state_dict`` …) is what the recipes' schedulers and checkpoints use;
    hyper-parameters live in the first store's group and are copied to the others before every step."""

    def __init__(self, device: torch.device, specs: Sequence[StoreSpec], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 shard_group: Any = None):
        self.device = device
        self.specs = [s for s in specs if s.params]
        self.shard_group = shard_group  # ranks that hold *different* local shards (tensor- / expert-parallel group); used by checkpoints
        self.flats: List[FlatParameters] = []
        self.opts: List[ShardedAdamW] = []
        for spec in self.specs:
            world, rank = spec.size()
            flat = FlatParameters(spec.params, world, device, spec.group, min_bucket_numel=1 << 22)
            if device.type == "cuda":
                torch.cuda.empty_cache()  # the parameters' old storage goes back to the driver before the next store is allocated
            self.flats.append(flat)
            self.opts.append(ShardedAdamW(flat, rank, world, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, group=None if spec.group is SOLO else spec.group))
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.step_count = 0

    # torch.optim-like surface ----------------------------------------------------------------
    torch_optimizer = property(lambda self: self)

    @property
    def param_groups(self) -> List[Dict[str, Any]]:
        return self.opts[0].param_groups

    def _sync_hyper_parameters(self) -> None:
        lead = self.opts[0].param_groups[0]
        for o in self.opts[1:]:
            for k, v in lead.items():
                if k != "params":
                    o.param_groups[0][k] = v

    def zero_grad(self, set_to_none: bool = True) -> None:
        for f in self.flats:
            f.reset_grad_flags()
            for p in f.params:
                p.grad = None

    def state_dict(self) -> Dict[str, Any]:
        return {"stores": {spec.name: o.state_dict() for spec, o in zip(self.specs, self.opts)}}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        for spec, o in zip(self.specs, self.opts):
            o.load_state_dict(sd["stores"][spec.name])
        self.step_count = self.opts[0].step_count

    def full_state_dict(self, is_rank_zero: bool = True, group=None) -> Dict[str, Any]:
        """Checkpoint form (collective).  A store summed over every rank is identical everywhere and is saved once; a local
        store differs per shard position, so the full moments of every position of the shard group are collected."""
        out: Dict[str, Any] = {"stores": {}}
        for spec, o in zip(self.specs, self.opts):
            full = o.full_state_dict(True, group=o.group)  # every rank of the store's group gets the full moments of its shard
            if spec.group is None:
                out["stores"][spec.name] = full
                continue
            n = dist.get_world_size(self.shard_group) if (dist.is_initialized() and self.shard_group is not SOLO) else 1
            per_position: List[Any] = [None] * n
            if n > 1:
                dist.all_gather_object(per_position, full, group=self.shard_group)
            else:
                per_position[0] = full
            out["stores"][spec.name] = {"shard_positions": per_position}
        return out if is_rank_zero else {}

    def load_full_state_dict(self, sd: Dict[str, Any]) -> None:
        for spec, o in zip(self.specs, self.opts):
            entry = sd["stores"][spec.name]
            if "shard_positions" in entry:
                n = dist.get_world_size(self.shard_group) if (dist.is_initialized() and self.shard_group is not SOLO) else 1
                if len(entry["shard_positions"]) != n:
                    raise ValueError("optimizer checkpoint was written with a different tensor- / expert-parallel size")
                pos = dist.get_rank(self.shard_group) if n > 1 else 0
                entry = entry["shard_positions"][pos]
            o.load_full_state_dict(entry)
        self.step_count = self.opts[0].step_count

    # step ------------------------------------------------------------------------------------
    def collect_grads(self) -> None:
        for f in self.flats:
            f.collect_autograd_grads()

    def step(self, grad_scale: Union[float, torch.Tensor] = 1.0, max_grad_norm: Optional[float] = None, group=None) -> None:
        """``group``: the whole job (the clipping norm is summed over it).  Gradients must already sit in the flat buffers
        (:meth:`collect_grads`) and, on CUDA, every rank's buffers must be complete (the caller's barrier)."""
        self._sync_hyper_parameters()
        self.step_count += 1
        for o in self.opts:
            o.begin_step(grad_scale, max_grad_norm)
        try:
            for o in self.opts:
                o.reduce_all()
            total = None
            if max_grad_norm is not None:
                total = torch.stack([o.local_sumsq().reshape(()) for o in self.opts]).sum()
                if dist.is_initialized() and dist.get_world_size(group) > 1:
                    dist.all_reduce(total, group=group)
        except BaseException:
            for o in self.opts:
                o._open = None
            raise
        for o in self.opts:
            o.finish(total)
        self.last_grad_norm = self.opts[0].last_grad_norm

    def close(self) -> None:
        for f in self.flats:
            f.close()
        self.flats = []
