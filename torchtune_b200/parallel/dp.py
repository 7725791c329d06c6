"""Data parallelism with resident parameters and a sharded, fused optimizer step.

Design (sized for 180 GB of HBM per GPU): every rank keeps the full bf16 parameters and a
full bf16 gradient buffer as two *flat* peer-visible allocations; optimizer moments are
sharded (rank r owns elements ``[r·S, (r+1)·S)``).  One step of communication is a single
kernel per rank (``ttb_dp_reduce_adamw_bcast``): pull the gradient slices of all peers,
reduce in fp32, AdamW on the owned slice, push the new parameters to all peers.  Compared
with the reference's FSDP2 path (per-layer all-gather in forward and backward, per-layer
reduce-scatter, then a separate scale pass and optimizer step —
torchtune/training/_distributed.py:661-714, recipes/full_finetune_distributed.py:1030-1050)
this moves 2 instead of 3 model-sized messages per step, keeps nothing on the critical path
of the layers, and reduces in fp32 while sending bf16.

Models that do not fit resident use the ZeRO-3 sharder in :mod:`.fsdp`.
On CPU (gloo) the same interface is implemented with ``all_reduce`` so the host-side logic
is testable without GPUs.
"""
from __future__ import annotations

import ctypes
import math
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from ..ops import reference as _ref
from .fabric import PeerBuffer

_ALIGN = 2048  # elements; keeps every shard and every parameter offset 16-byte aligned


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


class FlatParameters:
    """Re-homes the trainable parameters of ``model`` into one flat buffer (and gives each a
    same-shaped window of a flat gradient buffer, exposed as ``param._grad_buffer``)."""

    def __init__(self, params: List[Tuple[str, nn.Parameter]], world: int, device: torch.device, group=None):
        dtypes = {p.dtype for _, p in params}
        if len(dtypes) != 1:
            raise ValueError(f"all trainable parameters must share one dtype, found {dtypes}")
        self.dtype = dtypes.pop()
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.offsets: List[int] = []
        cursor = 0
        for p in self.params:
            self.offsets.append(cursor)
            cursor += _round_up(p.numel(), 8)
        self.shard = _round_up(-(-cursor // world), _ALIGN)
        self.total = self.shard * world
        esize = torch.empty(0, dtype=self.dtype).element_size()
        self.param_buf = PeerBuffer(self.total * esize, device, group)
        self.grad_buf = PeerBuffer(self.total * esize, device, group)
        self.flat_param = self.param_buf.tensor(self.dtype, self.total)
        self.flat_grad = self.grad_buf.tensor(self.dtype, self.total)
        with torch.no_grad():
            for p, off in zip(self.params, self.offsets):
                window = self.flat_param[off : off + p.numel()].view(p.shape)
                window.copy_(p.data)
                p.data = window
                p._grad_buffer = self.flat_grad[off : off + p.numel()].view(p.shape)
                p._grad_written = False
        if device.type == "cuda":
            from ..ops import _cuda

            for p in self.params:
                _cuda.register_grad_window(p)

    def collect_autograd_grads(self) -> None:
        """Move gradients that autograd produced as separate tensors into the flat buffer and
        zero the windows nothing wrote to."""
        for p in self.params:
            if p.grad is not None:
                if p._grad_written:
                    p._grad_buffer.add_(p.grad)
                else:
                    p._grad_buffer.copy_(p.grad)
                p._grad_written = True
                p.grad = None
            elif not p._grad_written:
                p._grad_buffer.zero_()

    def reset_grad_flags(self) -> None:
        for p in self.params:
            p._grad_written = False

    def close(self) -> None:
        self.param_buf.close()
        self.grad_buf.close()


class ShardedAdamW:
    """AdamW over a :class:`FlatParameters` store; this rank updates shard ``rank`` only and
    the fused kernel distributes the result."""

    def __init__(self, flat: FlatParameters, rank: int, world: int, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2):
        self.flat, self.rank, self.world = flat, rank, world
        self.param_groups = [dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, params=flat.params)]
        dev = flat.flat_param.device
        self.exp_avg = torch.zeros(flat.shard, dtype=flat.dtype, device=dev)
        self.exp_avg_sq = torch.zeros(flat.shard, dtype=flat.dtype, device=dev)
        self.step_count = 0
        self._gsum: Optional[torch.Tensor] = None
        self.last_grad_norm: Optional[torch.Tensor] = None

    # torch.optim-like surface used by schedulers / loggers
    @property
    def torch_optimizer(self):
        return self

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.reset_grad_flags()

    def state_dict(self) -> Dict[str, Any]:
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(saved)

    def full_state_dict(self, is_rank_zero: bool = True, group=None) -> Dict[str, Any]:
        """Moments of the whole model as one flat CPU tensor each plus the parameter layout, so a
        checkpoint written at one world size can be read at another."""
        flat = self.flat
        out = {}
        for key, shard in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            if self.world > 1:
                parts = [torch.empty_like(shard) for _ in range(self.world)]
                dist.all_gather(parts, shard, group=group)
                full = torch.cat(parts)
            else:
                full = shard
            out[key] = full.cpu() if is_rank_zero else None
        if not is_rank_zero:
            return {}
        out["step"] = self.step_count
        out["layout"] = {"names": list(flat.names), "offsets": list(flat.offsets), "numels": [p.numel() for p in flat.params]}
        out["param_groups"] = [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]
        return out

    def load_full_state_dict(self, sd: Dict[str, Any]) -> None:
        flat = self.flat
        layout = sd.get("layout")
        if layout is not None and (list(layout["names"]) != list(flat.names) or list(layout["numels"]) != [p.numel() for p in flat.params]):
            raise ValueError("optimizer checkpoint was written for a different set of trainable parameters")
        self.step_count = int(sd["step"])
        begin = self.rank * flat.shard
        for key, shard in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            full = sd[key]
            shard.zero_()
            end = min(begin + flat.shard, full.numel())
            if end > begin:
                shard[: end - begin].copy_(full[begin:end])
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(saved)

    def step(self, grad_scale: Union[float, torch.Tensor] = 1.0, max_grad_norm: Optional[float] = None, group=None) -> None:
        g = self.param_groups[0]
        self.step_count += 1
        b1, b2 = g["betas"]
        inv_bc1 = 1.0 / (1.0 - b1**self.step_count)
        inv_sqrt_bc2 = 1.0 / math.sqrt(1.0 - b2**self.step_count)
        flat = self.flat
        begin = self.rank * flat.shard
        self.last_grad_norm = None
        if flat.flat_param.is_cuda:
            self._step_cuda(grad_scale, max_grad_norm, g, begin, inv_bc1, inv_sqrt_bc2, group)
        else:
            self._step_host(grad_scale, max_grad_norm, g, begin, group)

    def _step_cuda(self, grad_scale, max_grad_norm, g, begin, inv_bc1, inv_sqrt_bc2, group) -> None:
        from ..ops._lib import check, lib, stream_ptr

        L = lib()
        _declare_dp(L)
        flat = self.flat
        scale_dev, scale_host = (grad_scale.to(torch.float32).reshape(1), 1.0) if isinstance(grad_scale, torch.Tensor) else (None, float(grad_scale))
        b1, b2 = g["betas"]
        grads, params = flat.grad_buf.pointer_array(), flat.param_buf.pointer_array()

        def launch(mode: int, sdev, shost, gsum=None, partials=None):
            check(
                L.ttb_dp_reduce_adamw_bcast(grads, params, self.world, self.rank, begin, flat.shard, self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), None if gsum is None else gsum.data_ptr(), None if partials is None else partials.data_ptr(), None if sdev is None else sdev.data_ptr(), shost, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"], inv_bc1, inv_sqrt_bc2, mode, stream_ptr()),
                "dp_reduce_adamw_bcast",
            )

        if max_grad_norm is None:
            launch(0, scale_dev, scale_host)
            return
        if self._gsum is None:
            self._gsum = torch.empty(flat.shard, dtype=torch.float32, device=flat.flat_param.device)
        partials = torch.empty(L.ttb_dp_grid(), dtype=torch.float32, device=flat.flat_param.device)
        launch(1, None, 1.0, self._gsum, partials)
        sumsq = partials.sum()
        if self.world > 1:
            dist.all_reduce(sumsq, group=group)
        s = scale_dev if scale_dev is not None else torch.tensor([scale_host], device=sumsq.device)
        norm = sumsq.sqrt() * s
        self.last_grad_norm = norm.reshape(())
        coef = torch.clamp(float(max_grad_norm) / (norm + 1e-6), max=1.0) * s
        launch(2, coef.reshape(1).float(), 1.0, self._gsum)

    def _step_host(self, grad_scale, max_grad_norm, g, begin, group) -> None:
        """gloo implementation of the same algorithm (sum of all ranks' gradients in fp32,
        update of the owned shard, broadcast of the result)."""
        flat = self.flat
        gsum = flat.flat_grad.float()
        if self.world > 1:
            dist.all_reduce(gsum, group=group)
        scale = float(grad_scale) if not isinstance(grad_scale, torch.Tensor) else float(grad_scale.item())
        if max_grad_norm is not None:
            norm = gsum.norm() * scale
            self.last_grad_norm = norm
            scale *= float(torch.clamp(float(max_grad_norm) / (norm + 1e-6), max=1.0))
        sl = slice(begin, begin + flat.shard)
        b1, b2 = g["betas"]
        new = flat.flat_param[sl].clone()
        _ref.adamw_step(new, gsum[sl], self.exp_avg, self.exp_avg_sq, self.step_count, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"], scale)
        if self.world > 1:
            gathered = [torch.empty_like(new) for _ in range(self.world)]
            dist.all_gather(gathered, new, group=group)
            flat.flat_param.copy_(torch.cat(gathered))
        else:
            flat.flat_param[sl].copy_(new)


def _declare_dp(L) -> None:
    if getattr(L, "_dp_declared", False):
        return
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    L.ttb_dp_reduce_adamw_bcast.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, i64, i64, vp, vp, vp, vp, vp, f32, f32, f32, f32, f32, f32, f32, f32, i32, vp]
    L.ttb_dp_reduce_adamw_bcast.restype = i32
    L.ttb_dp_grid.restype = i32
    L._dp_declared = True


class DataParallelEngine:
    """Owns the flat stores, the wgrad side stream and the step protocol.

    Step protocol (all on the training stream, so ordering is stream order):
      backward … → ``all_reduce_sum_(n_tokens, …)``  — also the cross-rank barrier that tells
      every rank all gradient buffers are final → fused reduce/AdamW/broadcast kernel →
      small all-reduce as the closing barrier (new parameters have landed everywhere and
      nobody still reads the old gradients).
    """

    def __init__(self, device: torch.device, group=None):
        self.device = device
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.flat: Optional[FlatParameters] = None
        self._barrier_token = torch.zeros(1, device=device if device.type == "cuda" else "cpu")

    # sizes the recipes ask for ------------------------------------------------------------
    dp_size = property(lambda self: self.world)
    dp_rank = property(lambda self: self.rank)
    non_data_parallel_size = 1
    min_seq_len_divisor = 1

    def prepare(self, model: nn.Module) -> nn.Module:
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.flat = FlatParameters(named, self.world, self.device, self.group)
        if self.device.type == "cuda":
            from ..ops import _cuda

            _cuda.enable_direct_wgrad(True)
        return model

    def build_optimizer(self, model: nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, **_: Any) -> ShardedAdamW:
        if self.flat is None:
            raise RuntimeError("call prepare(model) first")
        return ShardedAdamW(self.flat, self.rank, self.world, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def all_reduce_sum_(self, *tensors: torch.Tensor) -> None:
        if self.world == 1:
            return
        if len(tensors) == 1:
            dist.all_reduce(tensors[0], group=self.group)
            return
        packed = torch.stack([t.reshape(()).to(torch.float32) for t in tensors])
        dist.all_reduce(packed, group=self.group)
        for t, v in zip(tensors, packed):
            t.copy_(v)

    def barrier(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._barrier_token, group=self.group)

    def optimizer_step(self, model: nn.Module, optimizer: ShardedAdamW, grad_scale, clip_grad_norm: Optional[float] = None):
        if self.device.type == "cuda":
            from ..ops import _cuda

            _cuda.join_wgrad_stream()
        self.flat.collect_autograd_grads()
        if self.world > 1 and self.device.type == "cuda":
            self.barrier()  # every rank's gradient buffer is complete
        optimizer.step(grad_scale=grad_scale, max_grad_norm=clip_grad_norm, group=self.group)
        if self.world > 1 and self.device.type == "cuda":
            self.barrier()  # pushes have landed; gradients may be overwritten
        optimizer.zero_grad()
        return optimizer.last_grad_norm

    def shutdown(self) -> None:
        if self.flat is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.barrier()
            self.flat.close()
            self.flat = None
