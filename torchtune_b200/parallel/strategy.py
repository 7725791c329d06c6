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


class TensorParallelOptimizer:
    """A ``torch.optim`` optimizer over the local (sharded + replicated) parameters of a tensor-parallel model:
    gradients of replicated parameters are summed over the group first; the clipping norm counts sharded
    parameters on every rank and replicated ones once."""

    def __init__(self, strategy: "ParallelStrategy", model: nn.Module, optimizer: torch.optim.Optimizer):
        self.strategy, self.model, self.optimizer = strategy, model, optimizer
        self.last_grad_norm: Optional[torch.Tensor] = None

    torch_optimizer = property(lambda self: self.optimizer)
    param_groups = property(lambda self: self.optimizer.param_groups)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd) -> None:
        self.optimizer.load_state_dict(sd)

    def full_state_dict(self, is_rank_zero: bool = True, group=None):
        """Optimizer state of *this rank's shard*; resuming requires the same tensor-parallel size."""
        return {"tp_rank_states": self._gather_states()} if is_rank_zero else (self._gather_states() and {})

    def _shard_group(self):
        """(group, size, rank) over which the model is split: the tensor- or expert-parallel group (under a dp × tp or dp × ep
        mesh the replicas hold identical shards and optimizer state), every rank otherwise."""
        ctx = self.strategy.tp if self.strategy.tp is not None else self.strategy.ep
        if ctx is not None:
            return ctx.group, ctx.world, ctx.rank
        return None, self.strategy.world, self.strategy.rank

    def _gather_states(self):
        group, world, _ = self._shard_group()
        states = [None] * world
        if world > 1:
            dist.all_gather_object(states, self.optimizer.state_dict(), group=group)
        else:
            states[0] = self.optimizer.state_dict()
        return states

    def load_full_state_dict(self, sd) -> None:
        _, world, rank = self._shard_group()
        states = sd.get("tp_rank_states")
        if states is None or len(states) != world:
            raise ValueError("optimizer checkpoint was written with a different tensor-parallel size")
        self.optimizer.load_state_dict(states[rank])

    def step(self, grad_scale=1.0, max_grad_norm: Optional[float] = None, group=None) -> None:
        model = self.model
        model.sync_replicated_grads()
        params = [p for p in model.parameters() if p.grad is not None]
        scale = grad_scale if isinstance(grad_scale, torch.Tensor) else torch.tensor(float(grad_scale), device=params[0].device)
        for p in params:
            p.grad.mul_(scale.to(p.grad.dtype))
        self.last_grad_norm = None
        if max_grad_norm is not None:
            replicated = {id(p) for p in model._replicated}
            sharded_sq = sum((p.grad.float().pow(2).sum() for p in params if id(p) not in replicated), torch.zeros((), device=params[0].device))
            repl_sq = sum((p.grad.float().pow(2).sum() for p in params if id(p) in replicated), torch.zeros((), device=params[0].device))
            group, world, _ = self._shard_group()
            if world > 1:
                dist.all_reduce(sharded_sq, group=group)
            norm = (sharded_sq + repl_sq).sqrt()
            self.last_grad_norm = norm
            coef = torch.clamp(float(max_grad_norm) / (norm + 1e-6), max=1.0)
            for p in params:
                p.grad.mul_(coef.to(p.grad.dtype))
        self.optimizer.step()
        after = getattr(model, "after_optimizer_step", None)
        if after is not None:
            after()


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
        self.ep_dim = int(get("expert_parallel_dim", 1) or 1)
        if self.ep_dim > 1 and (world % self.ep_dim or self.dims.tp_enabled):
            raise NotImplementedError("expert_parallel_dim > 1 must divide the world size and does not combine with tensor parallelism (use expert tensor parallelism: tensor_parallel_dim on an MoE model)")
        if self.dims.cp_enabled and (self.dims.tp_enabled or self.ep_dim > 1):
            raise NotImplementedError("context_parallel_dim > 1 combines with data parallelism only (not with tensor or expert parallelism)")
        super().__init__(device=device, group=None)
        self.tp = None  # TensorParallelContext, created in shard_model
        self.ep = None  # ExpertParallelContext, created in shard_model
        self.cp = None  # ContextParallelContext, created in shard_model
        self._replica_group = None  # ranks holding the same tensor- / expert-parallel shard (None: a single replica)
        self._stores = None  # MultiStoreAdamW of a sharded model (fused optimizer over two flat stores)
        self.zero3 = None  # ShardedWeightContext: linear weights sharded, fused weight-gather GEMM (`shard_parameters: linear`, LoRA bases)
        self.z3 = None  # Zero3Engine: every trainable parameter sharded (`shard_parameters: True` with an AdamW optimizer)
        self._shard_parameters = bool(get("shard_parameters", False)) and str(get("shard_parameters")).lower() not in ("false", "none", "0", "")
        self._shard_mode = str(get("shard_parameters", "")).lower()
        if (self._shard_parameters or self._shard_mode == "linear") and (self.dims.tp_enabled or self.ep_dim > 1 or self.dims.cp_enabled):
            raise NotImplementedError("shard_parameters combines with plain data parallelism only")
        self._cfg = cfg
        self._cpu_offload = bool(get("fsdp_cpu_offload", False))

    # sizes -------------------------------------------------------------------------------
    @property
    def non_data_parallel_size(self) -> int:  # type: ignore[override]
        return self.dims.non_data_parallel_size

    @property
    def min_seq_len_divisor(self) -> int:  # type: ignore[override]
        return self.dims.min_seq_len_divisor

    # data-parallel coordinates: with tensor parallelism every rank reads the same batch ------------
    @property
    def dp_size(self) -> int:  # type: ignore[override]
        # the ranks of one tensor- or context-parallel group (consecutive ranks) read the same batch
        return self.world // (self.dims.tp * self.dims.cp)  # (replicate × shard: every data-parallel rank reads its own batch)

    @property
    def dp_rank(self) -> int:  # type: ignore[override]
        return self.rank // (self.dims.tp * self.dims.cp)

    def _attach_context_parallel(self, model: nn.Module) -> None:
        """Context-parallel groups are runs of ``cp`` consecutive ranks; for parameters they are data-parallel ranks (every
        rank's gradient covers its own tokens and the resident engine sums over all ranks)."""
        from .cp import ContextParallelContext, context_parallelize

        cp = self.dims.cp
        group = None
        if cp != self.world:
            for g in range(self.world // cp):  # every rank creates every group, in the same order
                ranks = list(range(g * cp, (g + 1) * cp))
                handle = dist.new_group(ranks)
                if self.rank in ranks:
                    group = handle
        self.cp = ContextParallelContext(group, world=cp, rank=self.rank % cp)
        context_parallelize(model, self.cp)

    def _tp_max_rows(self, cfg, model: nn.Module) -> int:
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
        explicit = get("tensor_parallel_max_tokens")
        if explicit:
            return -(-int(explicit) // self.dims.tp)
        seq = None
        for section in ("tokenizer", "dataset"):
            sec = get(section)
            if sec is not None and hasattr(sec, "get"):
                seq = seq or sec.get("max_seq_len") or sec.get("seq_len")
        seq = int(seq or getattr(model, "max_seq_len", 2048))
        return -(-(int(get("batch_size", 1)) * seq) // self.dims.tp)

    def _shard_model_tp(self, model: nn.Module, cfg, prepare_layer=None) -> nn.Module:
        from ..training.memory import CheckpointedLayer
        from .tp import TensorParallelContext
        from .tp_model import tensor_parallelize

        core = model
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
        plan_cfg = get("tensor_parallel_plan")
        if plan_cfg is not None:
            # the layout is built into the engine; a plan named by the config is checked against it, never silently ignored
            from .. import config
            from ..models.llama3._parallelism import validate_tp_plan

            validate_tp_plan(config.instantiate(plan_cfg) if hasattr(plan_cfg, "get") and plan_cfg.get("_component_") else dict(plan_cfg))
        width = core.tok_embeddings.embedding_dim
        tp_group = dp_group = None
        if self.dims.tp != self.world:
            # dp × tp mesh, tensor-parallel ranks consecutive (they share NVLink peer buffers); the replicas of one shard
            # (same tensor-parallel rank) form the data-parallel group that sums its gradients
            groups = self.dims.build_groups(("dp", "tp"))
            tp_group, dp_group = groups["tp"], groups["dp"]
        self.tp = TensorParallelContext(self.device, tp_group, max_rows_per_rank=self._tp_max_rows(cfg, core), max_width=width)
        ac = any(isinstance(layer, CheckpointedLayer) for layer in core.layers)
        out = tensor_parallelize(core, self.tp, activation_checkpointing=ac, prepare_layer=prepare_layer)
        out.set_data_parallel_group(dp_group, self.world // self.dims.tp)
        self._replica_group = dp_group
        return out

    def _shard_model_ep(self, model: nn.Module, cfg, prepare_layer=None) -> nn.Module:
        """Experts spread over the ranks (every rank keeps its own batch: expert parallel ranks are data parallel for the
        dense part, whose gradients are summed before the optimizer step)."""
        from ..modules.moe import MoE
        from .ep import ExpertParallelContext, expert_parallelize

        first = next((m for m in model.modules() if isinstance(m, MoE)), None)
        if first is None:
            raise ValueError("expert_parallel_dim > 1 needs a model with MoE layers")
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
        router = first.router
        # no reference to a MoE module may survive into expert_parallelize: it would keep that layer's full expert stacks alive
        # after they have been cut down to this rank's experts (4 GB per Scout layer)
        num_experts, router_dim, experts_per_token = router.num_experts, router.dim, router.experts_per_token
        del first, router
        tokens = self._tp_max_rows(cfg, model) * max(self.dims.tp, 1)
        ep, replicas = self.ep_dim, self.world // self.ep_dim
        ep_group = replica_group = None
        if replicas > 1:
            # several expert-parallel groups of consecutive ranks; the ranks with the same position in their group own the same
            # experts.  Every rank creates every group, in the same order.
            for g in range(replicas):
                ranks = list(range(g * ep, (g + 1) * ep))
                handle = dist.new_group(ranks)
                if self.rank in ranks:
                    ep_group = handle
            for j in range(ep):
                ranks = list(range(j, self.world, ep))
                handle = dist.new_group(ranks)
                if self.rank in ranks:
                    replica_group = handle
        self.ep = ExpertParallelContext(self.device, ep_group, num_experts=num_experts, dim=router_dim, max_pairs=tokens * experts_per_token,
                                        capacity_factor=get("expert_capacity_factor"))
        self._replica_group = replica_group
        return expert_parallelize(model, self.ep, replica_group, replicas, prepare_layer=prepare_layer)

    # model -------------------------------------------------------------------------------
    def shard_model(self, model: nn.Module, cfg, base_sd: Dict[str, Any], adapter_sd: Optional[Dict[str, Any]] = None, *, dtype: torch.dtype = torch.bfloat16, strict: bool = True) -> nn.Module:
        from ..training._distributed import materialize, validate_no_params_on_meta_device

        is_lora = not strict
        layerwise = None
        if (self.dims.tp_enabled or self.ep_dim > 1) and not is_lora and any(p.is_meta for p in model.parameters()):
            # a model built on the meta device is given storage layer by layer while it is sharded: it never exists in full
            from ..training._distributed import LayerwisePreparer

            layerwise = LayerwisePreparer(self.device, state_dict=base_sd)
            if self.dims.tp_enabled:
                return self._shard_model_tp(model, cfg, layerwise)
            return self._shard_model_ep(model, cfg, layerwise)
        if self._shard_parameters and self._wants_full_sharding(cfg, is_lora) and any(p.is_meta for p in model.parameters()):
            # every parameter sharded, model still without storage (`shard_parameters_layerwise: True`, for models whose bf16
            # parameters do not fit one GPU): each bucket's modules get storage and checkpoint values right before they are cut
            from ..training._distributed import LayerwisePreparer
            from .zero3 import Zero3Engine

            shard_group = replica_group = None
            if self.dims.dp_replicate > 1:
                groups = self.dims.build_groups(("dp_shard", "dp_replicate"))
                shard_group, replica_group = groups["dp_shard"], groups["dp_replicate"]
            self.z3 = Zero3Engine(self.device, shard_group, replica_group)
            model = self.z3.prepare(model, prepare_layer=LayerwisePreparer(self.device, state_dict=base_sd))
            validate_no_params_on_meta_device(model)
            if self.rank == 0:
                _log.info(f"ZeRO-3 engine: every trainable parameter is sharded over {self.world} ranks ({self.z3.nb} buckets, {self.z3.sp.shard} elements per rank), built layer by layer")
            return model
        presharded = None
        if self._shard_parameters and not self._wants_full_sharding(cfg, is_lora) and any(t.is_meta for t in list(model.parameters()) + list(model.buffers())):
            # a base larger than one GPU (dense or 4-bit): this rank's rows of every weight go from the checkpoint straight into the
            # peer-visible store (parts of a 4-bit base get their storage) before anything else exists, so no whole weight ever does
            from .fsdp import shard_linear_weights

            get_ = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
            model = shard_linear_weights(model, self.device, None, min_numel=int(get_("shard_parameters_min_numel", 1 << 16)), state_dict=base_sd)
            presharded = set(model._sharded_keys)
            base_sd = {k: v for k, v in base_sd.items() if k not in presharded}
        materialize(model, self.device)
        if is_lora:
            from ..modules.peft import validate_missing_and_unexpected_for_lora

            base_missing, base_unexpected = model.load_state_dict(base_sd, strict=False)
            if presharded:
                base_missing = [k for k in base_missing if k not in presharded]
            lora_missing = lora_unexpected = None
            if adapter_sd is not None:
                lora_missing, lora_unexpected = model.load_state_dict(adapter_sd, strict=False)
            validate_missing_and_unexpected_for_lora(
                state_dict_keys=list(model.state_dict().keys()), base_missing=base_missing, base_unexpected=base_unexpected, lora_missing=lora_missing, lora_unexpected=lora_unexpected
            )
            if adapter_sd is None:
                # fresh adapters are drawn here, in module order from the job's seed, so that their values do not depend on how the
                # model came to exist (built on the device, where the throw-away base weights also consume random numbers, or on
                # the meta device)
                with torch.random.fork_rng(devices=[self.device] if self.device.type == "cuda" else []):
                    torch.manual_seed(torch.initial_seed())
                    for m in model.modules():
                        if callable(getattr(m, "adapter_params", None)) and callable(getattr(m, "initialize_parameters", None)):
                            m.initialize_parameters()
                for m in model.modules():
                    if hasattr(m, "initialize_dora_magnitude"):
                        m.initialize_dora_magnitude()
        elif presharded:
            missing, unexpected = model.load_state_dict(base_sd, strict=False)
            left = [k for k in missing if k not in presharded]
            if left or unexpected:
                raise RuntimeError(f"checkpoint does not match the model: missing {left[:4]}, unexpected {list(unexpected)[:4]}")
        else:
            model.load_state_dict(base_sd, strict=True)
        validate_no_params_on_meta_device(model)
        if presharded is not None:
            model.refresh_replicated()
        if self.dims.tp_enabled:
            if is_lora:
                raise NotImplementedError("tensor parallelism is implemented for full fine-tuning")
            return self._shard_model_tp(model, cfg)
        if self.ep_dim > 1:
            if is_lora:
                raise NotImplementedError("expert parallelism is implemented for full fine-tuning")
            return self._shard_model_ep(model, cfg)
        if self._shard_parameters and self._wants_full_sharding(cfg, is_lora):
            from .zero3 import Zero3Engine

            if self.world > 1:  # identical initial values on every rank before they are cut into shards
                for p in model.parameters():
                    if p.device.type == "cpu" and p.dtype == torch.bfloat16:
                        tmp = p.data.float()
                        dist.broadcast(tmp, src=0)
                        p.data.copy_(tmp)
                    else:
                        dist.broadcast(p.data, src=0)
            shard_group = replica_group = None
            if self.dims.dp_replicate > 1:
                # hybrid sharding: parameters are cut over runs of `dp_shard` consecutive ranks; the ranks at the same position
                # of every run hold the same slices and sum their reduced gradients once per step
                groups = self.dims.build_groups(("dp_shard", "dp_replicate"))
                shard_group, replica_group = groups["dp_shard"], groups["dp_replicate"]
            self.z3 = Zero3Engine(self.device, shard_group, replica_group)
            model = self.z3.prepare(model)
            if self.rank == 0:
                _log.info(f"ZeRO-3 engine: every trainable parameter is sharded over {self.world} ranks ({self.z3.nb} buckets, {self.z3.sp.shard} elements per rank)")
            return model
        if self._shard_parameters:
            from .fsdp import shard_linear_weights

            get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
            if presharded is None:
                model = shard_linear_weights(model, self.device, None, min_numel=int(get("shard_parameters_min_numel", 1 << 16)))
            self.zero3 = model._sw
            if is_lora and self.world > 1:
                # adapters are initialised with rank-dependent seeds: rank 0's values win
                for p in model._replicated:
                    if p.requires_grad:
                        if p.device.type == "cpu" and p.dtype == torch.bfloat16:
                            tmp = p.data.float()
                            dist.broadcast(tmp, src=0)
                            p.data.copy_(tmp)
                        else:
                            dist.broadcast(p.data, src=0)
            return model
        self.prepare(model)
        if self.dims.cp_enabled:
            self._attach_context_parallel(model)
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

    def _wants_full_sharding(self, cfg, is_lora: bool) -> bool:
        """Every parameter sharded (ZeRO-3 engine) for full fine-tuning with an AdamW-family optimizer and one parameter dtype;
        ``shard_parameters: linear``, LoRA (whose frozen base is what needs sharding) and other optimizers keep the
        sharded-linear-weight path."""
        if is_lora or self._shard_mode == "linear":
            return False
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: d)
        opt = get("optimizer")
        target = opt.get("_component_", "torch.optim.AdamW") if hasattr(opt, "get") else "torch.optim.AdamW"
        target = target.replace("torchtune.", "torchtune_b200.", 1) if target.startswith("torchtune.") else target
        if get("optimizer_in_bwd", False):
            return False
        return target in _FUSED_ADAMW and not (hasattr(opt, "get") and (opt.get("amsgrad", False) or opt.get("maximize", False)))

    def wants_backward_overlap(self, optimizer) -> bool:
        if self.z3 is not None:
            return self.z3.wants_backward_overlap(optimizer)
        return super().wants_backward_overlap(optimizer)

    def arm_backward_overlap(self, optimizer, grad_scale, clip_grad_norm: Optional[float] = None) -> bool:
        if self.z3 is not None:
            return self.z3.arm_backward_overlap(optimizer, grad_scale, clip_grad_norm)
        return super().arm_backward_overlap(optimizer, grad_scale, clip_grad_norm)

    # optimizer ---------------------------------------------------------------------------
    def _store_specs(self, model: nn.Module):
        """The two flat stores of a sharded model: parameters every rank holds (summed over the job) and this rank's shards
        (summed over the ranks that hold the same shard)."""
        from .fabric import SOLO
        from .stores import StoreSpec

        replicated = {id(p) for p in model._replicated}
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        local_group = getattr(self, "_replica_group", None)
        if local_group is None:
            local_group = SOLO  # one replica of every shard (also: row shards whose gradients arrive already reduce-scattered)
        ctx = self.tp if self.tp is not None else self.ep
        shard_group = ctx.group if ctx is not None else None
        return [StoreSpec("replicated", [(n, p) for n, p in named if id(p) in replicated], None),
                StoreSpec("local", [(n, p) for n, p in named if id(p) not in replicated], local_group)], shard_group

    def build_optimizer(self, model: nn.Module, cfg_optimizer=None, opt_state: Optional[Dict[str, Any]] = None, **kwargs: Any):
        if self.z3 is not None:
            params = {k: v for k, v in cfg_optimizer.items() if k != "_component_"} if hasattr(cfg_optimizer, "items") else dict(kwargs)
            if isinstance(cfg_optimizer, (int, float)):
                params["lr"] = float(cfg_optimizer)
            opt = self.z3.build_optimizer(model, lr=float(params.get("lr", 1e-3)), betas=tuple(params.get("betas", (0.9, 0.999))), eps=float(params.get("eps", 1e-8)),
                                          weight_decay=float(params.get("weight_decay", 1e-2)))
            if opt_state:
                opt.load_full_state_dict(opt_state)
            return opt
        if self.tp is not None or self.ep is not None or self.zero3 is not None:
            from .. import config

            target = cfg_optimizer.get("_component_", "torch.optim.AdamW") if hasattr(cfg_optimizer, "get") else "torch.optim.AdamW"
            target = target.replace("torchtune.", "torchtune_b200.", 1) if target.startswith("torchtune.") else target
            params = {k: v for k, v in cfg_optimizer.items() if k != "_component_"} if hasattr(cfg_optimizer, "items") else dict(kwargs)
            dtypes = {p.dtype for p in model.parameters() if p.requires_grad}
            if self.zero3 is None and target in _FUSED_ADAMW and not params.get("amsgrad", False) and not params.get("maximize", False) and len(dtypes) == 1:
                # fused path: moments of the replicated parameters sharded over every rank, those of a shard over its replicas
                from .stores import MultiStoreAdamW

                specs, shard_group = self._store_specs(model)
                if self.device.type == "cuda":
                    from ..ops import _cuda

                    _cuda.enable_direct_wgrad(True)
                opt = MultiStoreAdamW(self.device, specs, lr=float(params.get("lr", 1e-3)), betas=tuple(params.get("betas", (0.9, 0.999))),
                                      eps=float(params.get("eps", 1e-8)), weight_decay=float(params.get("weight_decay", 1e-2)), shard_group=shard_group)
                self._stores = opt
                if opt_state:
                    opt.load_full_state_dict(opt_state)
                return opt
            opt = TensorParallelOptimizer(self, model, config.instantiate(cfg_optimizer, [p for p in model.parameters() if p.requires_grad]))
            if opt_state:
                opt.load_full_state_dict(opt_state)
            return opt
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
        if self.z3 is not None:
            return self.z3.optimizer_step(model, optimizer, grad_scale, clip)
        if self.tp is not None or self.ep is not None or self.zero3 is not None:
            from .stores import MultiStoreAdamW

            if isinstance(optimizer, MultiStoreAdamW):
                if self.device.type == "cuda":
                    from ..ops import _cuda

                    _cuda.join_wgrad_stream()
                optimizer.collect_grads()
                cuda_peers = self.world > 1 and self.device.type == "cuda"
                if cuda_peers:
                    self.barrier()  # every rank's gradient buffers are complete before any peer pulls from them
                optimizer.step(grad_scale=grad_scale, max_grad_norm=clip, group=self.group)
                if cuda_peers:
                    self.barrier()  # pushed parameters have landed everywhere; gradient buffers may be overwritten
                optimizer.zero_grad()
                return optimizer.last_grad_norm
            optimizer.step(grad_scale=grad_scale, max_grad_norm=clip)
            optimizer.zero_grad()
            return optimizer.last_grad_norm
        return super().optimizer_step(model, optimizer, grad_scale, clip)

    # state dicts -------------------------------------------------------------------------
    def gather_full_state_dict(self, model: nn.Module) -> Dict[str, Any]:
        from ..training._distributed import gather_cpu_state_dict

        if self.z3 is not None:
            full = self.z3.full_state_dict(model)  # collective: every rank gathers every bucket
            return full if self.rank == 0 else {}
        if self.tp is not None or self.ep is not None or self.zero3 is not None:
            full = model.full_state_dict()  # collective: every rank takes part
            return {k: v.cpu() for k, v in full.items()} if self.rank == 0 else {}

        return gather_cpu_state_dict(model, self.rank == 0, self.device)

    def gather_optimizer_state_dict(self, model: nn.Module, optimizer) -> Dict[str, Any]:
        return optimizer.full_state_dict(self.rank == 0, group=self.group)

    def shutdown(self) -> None:
        if self._stores is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.barrier()
            self._stores.close()
            self._stores = None
        if self.tp is not None:
            self.tp.close()
            self.tp = None
        if self.ep is not None:
            self.ep.close()
            self.ep = None
        if self.zero3 is not None:
            self.zero3.close()
            self.zero3 = None
        if self.z3 is not None:
            self.z3.shutdown()
            self.z3 = None
        super().shutdown()
        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()


def init_from_config(cfg, device: torch.device) -> ParallelStrategy:
    return ParallelStrategy(cfg, device)
