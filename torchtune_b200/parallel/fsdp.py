"""Sharded-parameter data parallelism (ZeRO-3 for the linear weights) with a fused weight all-gather → GEMM.

The reference shards every parameter with FSDP2 (torchtune/training/_distributed.py:661-714): each layer's flat parameter is
all-gathered before its forward and again before its backward, gradients are reduce-scattered, and the optimizer works on the
shards.  Here the large ``nn.Linear`` weights — which are practically all of a decoder's parameters — are sharded by output rows
over the ranks and live in one peer-visible store; everything else (norm scales, embeddings, small or odd-shaped linears) stays
replicated with its gradient summed before the optimizer step.

* forward: ``ttb_gemm_wg_bf16`` — the GEMM's copier warps pull the peers' weight shards over NVLink n-tile by n-tile into a
  reusable local workspace while the tensor cores already work on the n-tiles of the own shard; no separate all-gather, no
  per-layer collective on the critical path (shards only change at the optimizer step, so forward needs no barrier at all);
* backward: the weight is gathered again (NCCL all-gather into the workspace), ``dx = dy · W`` and ``dW = dyᵀ · x`` run as plain
  tcgen05 GEMMs and ``dW`` is reduce-scattered to the owners of the rows;
* memory per rank: ``1 / world`` of the linear weights, their gradients and optimizer state, plus one gathered weight.

Without CUDA (gloo) the same module runs on ``all_gather`` / ``all_reduce`` so the logic is testable on CPU.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .fabric import PeerBuffer

_BF16 = torch.bfloat16


def _declare(L) -> None:
    if getattr(L, "_wg_declared", False):
        return
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    L.ttb_gemm_wg_bf16.argtypes = [vp, ctypes.POINTER(vp), vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, vp, vp, vp]
    L.ttb_gemm_wg_bf16.restype = i32
    L._wg_declared = True


class ShardedWeightContext:
    """Peer-visible store for the weight shards of one model plus the workspace the gathered weight lands in."""

    def __init__(self, device: torch.device, group=None, *, store_numel: int, max_weight_numel: int, max_out_features: int):
        self.device, self.group = device, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cuda = device.type == "cuda"
        self._cursor = 0
        self._token = torch.zeros(1, device=device)
        if self.cuda:
            from ..ops._lib import lib

            _declare(lib())
            self.store = PeerBuffer(max(store_numel, 8) * 2, device, group)
            self.workspace = torch.empty(max(max_weight_numel, 8), dtype=_BF16, device=device)
            self.sync = torch.empty(2 + max_out_features // 64, dtype=torch.int32, device=device)

    def barrier(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def close(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            self.barrier()
            self.store.close()

    def place(self, shard: torch.Tensor) -> torch.Tensor:
        """Copy ``shard`` (``[rows, K]``) into the store and return the view that replaces it (same offset on every rank)."""
        if not self.cuda:
            return shard.detach().clone()
        n = shard.numel()
        view = self.store.tensor(_BF16, self._cursor + n)[self._cursor :].view(shard.shape)
        view.copy_(shard)
        self._cursor += (n + 7) // 8 * 8
        return view

    def _store_offset(self, shard: torch.Tensor) -> Optional[int]:
        """Element offset of ``shard`` inside the store (identical on every rank), or ``None`` if it lives elsewhere."""
        if not self.cuda:
            return None
        delta = shard.data_ptr() - self.store.local_ptr
        return delta // 2 if 0 <= delta < self.store.nbytes and delta % 16 == 0 else None

    # ------------------------------------------------------------------ forward: fused gather + GEMM
    def fusable(self, x2: torch.Tensor, shard: torch.Tensor) -> bool:
        rows, k = shard.shape
        n = rows * self.world
        bn = 256 if n > 128 else (128 if n > 64 else 64)
        return self.cuda and x2.dtype == _BF16 and shard.dtype == _BF16 and rows % bn == 0 and k % 8 == 0 and shard.is_contiguous() and self._store_offset(shard) is not None

    def linear(self, x2: torch.Tensor, shard: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        """``x2 @ concat_ranks(shard).T (+ bias)`` → ``[T, world·rows]``."""
        rows, k = shard.shape
        if not self.fusable(x2, shard):
            return F.linear(x2, self.gather(shard), bias)
        from ..ops._lib import check, err_word, lib, stream_ptr

        n = rows * self.world
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        out = torch.empty(x2.shape[0], n, dtype=_BF16, device=self.device)
        ptrs = (ctypes.c_void_p * self.world)(*[p + 2 * self._store_offset(shard) for p in self.store.peer_ptrs])
        check(lib().ttb_gemm_wg_bf16(x2.data_ptr(), ptrs, out.data_ptr(), self.workspace.data_ptr(), self.sync.data_ptr(), self.world, self.rank, rows, x2.shape[0], k,
                                     k, n, None if bias is None else bias.data_ptr(), err_word(self.device).data_ptr(), stream_ptr()), "gemm_wg")
        return out

    # ------------------------------------------------------------------ backward: plain collectives
    def gather(self, shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return shard
        rows, k = shard.shape
        if self.cuda and shard.dtype == _BF16:
            full = self.workspace[: self.world * rows * k].view(self.world * rows, k)
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
            return full
        src = shard.float() if shard.dtype == _BF16 else shard
        parts = [torch.empty_like(src) for _ in range(self.world)]
        dist.all_gather(parts, src.contiguous(), group=self.group)
        return torch.cat(parts).to(shard.dtype)

    def reduce_scatter_rows(self, full: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return full
        rows = full.shape[0] // self.world
        if self.cuda:
            out = torch.empty(rows, full.shape[1], dtype=full.dtype, device=full.device)
            dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
            return out
        f = full.float().contiguous()
        dist.all_reduce(f, group=self.group)
        return f[self.rank * rows : (self.rank + 1) * rows].to(full.dtype)


class _WeightGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, bias, sw: ShardedWeightContext):
        ctx.sw = sw
        ctx.save_for_backward(x, shard)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        return sw.linear(x2, shard, bias).view(*x.shape[:-1], shard.shape[0] * sw.world)

    @staticmethod
    def backward(ctx, dy):
        from .tp import _wgrad

        x, shard = ctx.saved_tensors
        sw = ctx.sw
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            w_full = sw.gather(shard)
            if dy2.is_cuda and dy2.dtype == _BF16:
                from ..ops._cuda import gemm

                dx = gemm(dy2 if dy2.is_contiguous() else dy2.contiguous(), w_full, b_mn=True)
            else:
                dx = dy2 @ w_full
            dx = dx.view(x.shape)
        if ctx.needs_input_grad[1]:
            dw = sw.reduce_scatter_rows(_wgrad(dy2, x2))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None


class ShardedLinear(nn.Module):
    """``nn.Linear`` whose weight rows are split over the ranks (``weight``: this rank's ``[out / world, in]`` rows)."""

    def __init__(self, lin: nn.Linear, sw: ShardedWeightContext, shard: Optional[torch.Tensor] = None):
        """``shard``: this rank's rows when ``lin`` has no storage (a model built on the meta device)."""
        super().__init__()
        self.sw = sw
        self.in_features, self.out_features = lin.in_features, lin.out_features
        rows = lin.out_features // sw.world
        if shard is None:
            shard = lin.weight.data[sw.rank * rows : (sw.rank + 1) * rows]
        self.weight = nn.Parameter(sw.place(shard), requires_grad=lin.weight.requires_grad)
        self.bias = lin.bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _WeightGatherLinear.apply(x, self.weight, self.bias, self.sw)

    def full_weight(self) -> torch.Tensor:
        return self.sw.gather(self.weight.detach()).clone()


class ShardedLoRALinear(nn.Module):
    """LoRA linear (``modules/peft/lora.py::LoRALinear``, dense base) whose *frozen* base weight is split by rows over the ranks;
    the rank-``r`` adapters stay replicated and their gradients are summed before the optimizer step.  The reference shards LoRA
    base weights through FSDP (recipes/lora_finetune_distributed.py:548); this is what lets a 70B bf16 base fit next to
    activations."""

    def __init__(self, lora: nn.Module, sw: ShardedWeightContext, shard: Optional[torch.Tensor] = None):
        super().__init__()
        self.sw = sw
        self.rank, self.alpha, self.in_dim, self.out_dim, self.use_bias = lora.rank, lora.alpha, lora.in_dim, lora.out_dim, lora.use_bias
        rows = lora.out_dim // sw.world
        if shard is None:
            shard = lora.weight.data[sw.rank * rows : (sw.rank + 1) * rows]
        self.weight = nn.Parameter(sw.place(shard), requires_grad=False)
        self.bias = lora.bias
        self.dropout, self.lora_a, self.lora_b = lora.dropout, lora.lora_a, lora.lora_b
        self.merged = False
        self.disabled = False

    def adapter_params(self):
        return ["lora_a.weight", "lora_b.weight"]

    def initialize_parameters(self) -> None:
        """Adapter initialisation for a module whose adapters were given storage after construction (meta-device build)."""
        from ..modules.peft.lora import _lora_a_init_params, _lora_b_init_params

        _lora_a_init_params(self.lora_a)
        _lora_b_init_params(self.lora_b)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops

        base = _WeightGatherLinear.apply(x, self.weight, self.bias, self.sw)
        if self.disabled:
            return base
        a = ops.linear(self.dropout(x), self.lora_a.weight)
        return base + (self.alpha / self.rank) * ops.linear(a, self.lora_b.weight)

    def full_weight(self) -> torch.Tensor:
        return self.sw.gather(self.weight.detach()).clone()


def _dims(m: nn.Module):
    """(out_features, in_features) of a module whose ``weight`` can be row-sharded, else ``None``."""
    if type(m).__name__ == "Linear" and isinstance(m, nn.Linear):
        return m.out_features, m.in_features
    if type(m).__name__ == "LoRALinear" and not getattr(m, "_quantize_base", False) and getattr(m, "weight", None) is not None:
        return m.out_dim, m.in_dim
    return None


def shard_nf4_bases(model: nn.Module, device: torch.device, group=None, *, min_numel: int = 1 << 16) -> int:
    """Cut every frozen 4-bit base weight (``LoRALinear(quantize_base=True)``, ``FrozenNF4Linear``) into one part per rank
    (:class:`~torchtune_b200.modules.low_precision.ShardedNF4Weight`); returns how many were cut.

    Works on a model built under ``torch.device('meta')`` as well: a part is then allocated directly, so the whole 4-bit weight
    never exists on this rank, and the values arrive when the checkpoint is loaded (each dense weight is coded as a whole and this
    rank's part kept).  Weights that do not split at a boundary of their scale groups stay whole."""
    from ..modules.low_precision import NF4Weight, ShardedNF4Weight

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return 0
    cut = 0
    for owner in list(model.modules()):
        full = getattr(owner, "nf4", None)
        if type(full) is not NF4Weight:
            continue
        out_dim, in_dim = full.shape
        if out_dim * in_dim < min_numel or not ShardedNF4Weight.divisible(out_dim, in_dim, world, full.block_size, full.scaler_block_size):
            continue
        if full.weight_nf4.is_meta:
            part = ShardedNF4Weight(out_dim, in_dim, rank=rank, world=world, group=group, block_size=full.block_size, scaler_block_size=full.scaler_block_size,
                                    dtype=full.dtype, device=device)
        else:
            part = ShardedNF4Weight.from_full(full, rank=rank, world=world, group=group)
        owner.nf4 = part
        cut += 1
    return cut


def shard_linear_weights(model: nn.Module, device: torch.device, group=None, *, min_numel: int = 1 << 16, exclude=("output",),
                         state_dict: Optional[Dict[str, torch.Tensor]] = None) -> nn.Module:
    """Replace every plain ``nn.Linear`` (and every dense-base ``LoRALinear``) with at least ``min_numel`` weights whose rows split
    evenly into whole n-tiles by a :class:`ShardedLinear` (:class:`ShardedLoRALinear`) (in place; module paths in ``exclude`` and
    the small adapter matrices inside LoRA modules are left alone) and attach ``_replicated``, ``sync_replicated_grads()``, ``after_optimizer_step()`` and
    ``full_state_dict()`` (checkpoint layout; collective) to ``model``.

    A model built on the meta device is sharded without ever holding a whole weight on the device: with ``state_dict`` (the full
    checkpoint, model-level keys) each target's rows for this rank are copied from there straight into the store, one weight at a
    time; ``model._sharded_keys`` then names the checkpoint keys that have been consumed, and everything else is still to be
    given storage and loaded by the caller."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    shard_nf4_bases(model, device, group, min_numel=min_numel)  # 4-bit bases: parts of the codes, gathered and expanded per use

    def eligible(m: nn.Module) -> bool:
        dims = _dims(m)
        if dims is None or m.weight.numel() < min_numel:
            return False
        out_features, in_features = dims
        if device.type != "cuda":
            return out_features % world == 0
        rows = out_features // world
        bn = 256 if out_features > 128 else (128 if out_features > 64 else 64)
        return out_features % world == 0 and rows % bn == 0 and in_features % 8 == 0 and m.weight.dtype == _BF16

    # the output projection stays whole: the fused linear + cross-entropy loss reads its weight directly
    targets = [(parent, name, child) for pname, parent in model.named_modules() if not callable(getattr(parent, "adapter_params", None))
               for name, child in parent.named_children() if eligible(child) and (f"{pname}.{name}" if pname else name) not in exclude]
    paths = {id(child): (f"{pname}.{name}" if pname else name) for pname, parent in model.named_modules() for name, child in parent.named_children()}

    def checkpoint_key(child: nn.Module) -> Optional[str]:
        """Key of this module's weight in ``state_dict``: its module path, or that path without the ``layer.`` level that fusion
        layers leave out of their state dicts."""
        if state_dict is None:
            return None
        key = paths[id(child)] + ".weight"
        for cand in (key, key.replace(".layer.", ".")):
            if cand in state_dict:
                return cand
        return None

    # a weight without storage can only be sharded from a checkpoint value; one that has none stays whole (the caller gives it
    # storage and loads it like any other parameter)
    targets = [t for t in targets if not t[2].weight.is_meta or checkpoint_key(t[2]) is not None]
    store = sum(((c.weight.numel() // world) + 7) // 8 * 8 for _, _, c in targets)
    sw = ShardedWeightContext(device, group, store_numel=store, max_weight_numel=max((c.weight.numel() for _, _, c in targets), default=8),
                              max_out_features=max((_dims(c)[0] for _, _, c in targets), default=64))
    consumed = set()
    for parent, name, child in targets:
        shard = None
        if child.weight.is_meta:
            key = checkpoint_key(child)
            rows = _dims(child)[0] // world
            rank = dist.get_rank(group) if dist.is_initialized() else 0
            shard = state_dict[key][rank * rows : (rank + 1) * rows].to(device=device, dtype=child.weight.dtype)
            consumed.update((key, paths[id(child)] + ".weight"))  # as the checkpoint names it and as load_state_dict reports it
        setattr(parent, name, ShardedLinear(child, sw, shard) if isinstance(child, nn.Linear) else ShardedLoRALinear(child, sw, shard))
        if not child.weight.is_meta:
            child.weight.data = torch.empty(0, dtype=child.weight.dtype, device=child.weight.device)
    model._sharded_keys = consumed
    sharded = {id(m.weight) for m in model.modules() if isinstance(m, (ShardedLinear, ShardedLoRALinear))}
    def refresh_replicated() -> None:
        """Parameters that every rank holds whole.  Giving a meta-device parameter storage makes a new parameter object, so a
        caller that materialises the rest of the model after the sharding calls this again."""
        model._replicated = [p for p in model.parameters() if id(p) not in sharded]

    refresh_replicated()
    model.refresh_replicated = refresh_replicated
    model._sw = sw

    def sync_replicated_grads() -> None:
        grads = [p.grad for p in model._replicated if p.grad is not None]
        if not grads or sw.world == 1:
            return
        big = [g for g in grads if g.numel() >= (1 << 20) and g.is_cuda and g.is_contiguous()]
        for g in big:  # large tensors are reduced in place; the many small ones share one flat fp32 buffer
            dist.all_reduce(g, group=group)
        grads = [g for g in grads if not any(g is b for b in big)]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=group)
        off = 0
        for g in grads:
            g.copy_(flat[off : off + g.numel()].view_as(g))
            off += g.numel()

    def full_state_dict() -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        fulls = {f"{name}.weight": m.full_weight() for name, m in model.named_modules() if isinstance(m, (ShardedLinear, ShardedLoRALinear))}
        for k, v in model.state_dict().items():
            out[k] = fulls.get(k, v.detach())
        return out

    model.sync_replicated_grads = sync_replicated_grads
    model.after_optimizer_step = sw.barrier  # shards may be read by peers again only after every rank has updated its own
    model.full_state_dict = full_state_dict
    return model
