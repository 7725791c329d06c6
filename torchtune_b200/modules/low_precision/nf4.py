"""Owned NF4 storage for frozen base weights.

The reference delegates NF4 to an external tensor subclass (used at
torchtune/modules/peft/lora.py:83-87 and torchtune/modules/low_precision/nf4_linear.py:16-70).
Here the 4-bit codes and the double-quantised scales are ordinary module buffers:

* ``weight_nf4``      uint8 ``[out*in/2]``  two codes per byte (high nibble first)
* ``scaler_q``        int8  ``[n_blocks]``  per-block absmax, mean-centred, quantised
* ``scaler_factor``   fp32  ``[n_blocks / scaler_block_size]``
* ``scaler_mean``     fp32  scalar

``state_dict()`` exposes a single dense ``weight`` (dequantised, in ``dtype``) and
``load_state_dict`` accepts a dense ``weight`` and quantises it, so checkpoints stay in
the ordinary bf16 layout.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ...ops import reference as _ref


class NF4Weight(nn.Module):
    def __init__(
        self,
        out_dim: int,
        in_dim: int,
        block_size: int = 64,
        scaler_block_size: int = 256,
        dtype: torch.dtype = torch.bfloat16,
        device=None,
    ) -> None:
        super().__init__()
        n = out_dim * in_dim
        if n % block_size or (n // block_size) % scaler_block_size:
            raise ValueError(
                f"NF4 needs out*in ({n}) divisible by block_size*scaler_block_size ({block_size * scaler_block_size})"
            )
        self.shape: Tuple[int, int] = (out_dim, in_dim)
        self.block_size = block_size
        self.scaler_block_size = scaler_block_size
        self.dtype = dtype
        nb = n // block_size
        self.register_buffer("weight_nf4", torch.zeros(n // 2, dtype=torch.uint8, device=device), persistent=False)
        self.register_buffer("scaler_q", torch.zeros(nb, dtype=torch.int8, device=device), persistent=False)
        self.register_buffer(
            "scaler_factor", torch.ones(nb // scaler_block_size, dtype=torch.float32, device=device), persistent=False
        )
        self.register_buffer("scaler_mean", torch.zeros((), dtype=torch.float32, device=device), persistent=False)

    @torch.no_grad()
    def quantize_(self, dense: torch.Tensor) -> None:
        if tuple(dense.shape) != self.shape:
            raise ValueError(f"expected weight of shape {self.shape}, got {tuple(dense.shape)}")
        packed, sq, sf, mean = _encode(dense.to(self.weight_nf4.device), self.block_size, self.scaler_block_size)
        self.weight_nf4.copy_(packed)
        self.scaler_q.copy_(sq)
        self.scaler_factor.copy_(sf)
        self.scaler_mean.copy_(mean)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return _expand(self.weight_nf4, self.scaler_q, self.scaler_factor, self.scaler_mean, self.shape, self.block_size, self.scaler_block_size, dtype or self.dtype)

    def get_original_weight(self) -> torch.Tensor:
        return self.dequantize()

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers())


def _expand(packed, scaler_q, scaler_factor, scaler_mean, shape, block_size: int, scaler_block_size: int, target: torch.dtype) -> torch.Tensor:
    n = shape[0] * shape[1]
    if packed.is_cuda and target == torch.bfloat16 and n % 16 == 0 and block_size % 16 == 0:
        from ...ops import _cuda, cuda_ops_enabled

        if cuda_ops_enabled(packed):
            return _cuda.nf4_dequantize(packed, scaler_q, scaler_factor, scaler_mean, shape, block_size, scaler_block_size)
    return _ref.nf4_dequantize(packed, scaler_q, scaler_factor, scaler_mean, shape, block_size, scaler_block_size, target)


def _encode(dense: torch.Tensor, block_size: int, scaler_block_size: int):
    if dense.is_cuda and dense.dtype == torch.bfloat16 and block_size % 32 == 0:
        from ...ops import _cuda, cuda_ops_enabled

        if cuda_ops_enabled(dense):
            return _cuda.nf4_quantize(dense, block_size, scaler_block_size)
    return _ref.nf4_quantize(dense, block_size, scaler_block_size)


class ShardedNF4Weight(nn.Module):
    """One rank's part of an :class:`NF4Weight`: ``1/world`` of the codes and of the block scales, cut at a boundary of the scale
    groups so that the parts of all ranks, laid end to end, are exactly the buffers of the whole weight.

    ``dequantize()`` is a collective: it gathers the four small buffers (½ byte + 1/64 byte per weight, a quarter of what gathering
    bf16 would move) and expands them on this rank, so a frozen 4-bit base larger than one GPU — the 405B QLoRA configuration —
    costs each rank ``1/world`` of it plus one expanded weight at a time.  The reference gets the same effect by handing its NF4
    tensor subclass to FSDP (recipes/lora_finetune_distributed.py:548-575).  Every rank must reach each ``dequantize()`` in the
    same order, which the forward and backward of one model do."""

    def __init__(self, out_dim: int, in_dim: int, *, rank: int, world: int, group=None, block_size: int = 64, scaler_block_size: int = 256,
                 dtype: torch.dtype = torch.bfloat16, device=None) -> None:
        super().__init__()
        if not self.divisible(out_dim, in_dim, world, block_size, scaler_block_size):
            raise ValueError(f"a {out_dim} x {in_dim} NF4 weight does not split into {world} parts at scale-group boundaries")
        self.shape: Tuple[int, int] = (out_dim, in_dim)
        self.block_size, self.scaler_block_size, self.dtype = block_size, scaler_block_size, dtype
        self.rank, self.world, self.group = rank, world, group
        per = out_dim * in_dim // world
        self.register_buffer("weight_nf4", torch.zeros(per // 2, dtype=torch.uint8, device=device), persistent=False)
        self.register_buffer("scaler_q", torch.zeros(per // block_size, dtype=torch.int8, device=device), persistent=False)
        self.register_buffer("scaler_factor", torch.ones(per // block_size // scaler_block_size, dtype=torch.float32, device=device), persistent=False)
        self.register_buffer("scaler_mean", torch.zeros((), dtype=torch.float32, device=device), persistent=False)

    @staticmethod
    def divisible(out_dim: int, in_dim: int, world: int, block_size: int = 64, scaler_block_size: int = 256) -> bool:
        n = out_dim * in_dim
        return n % world == 0 and (n // world) % (block_size * scaler_block_size) == 0

    @classmethod
    def from_full(cls, full: NF4Weight, *, rank: int, world: int, group=None) -> "ShardedNF4Weight":
        part = cls(full.shape[0], full.shape[1], rank=rank, world=world, group=group, block_size=full.block_size, scaler_block_size=full.scaler_block_size,
                   dtype=full.dtype, device=full.weight_nf4.device)
        part._keep_own_part(full.weight_nf4, full.scaler_q, full.scaler_factor, full.scaler_mean)
        return part

    def _keep_own_part(self, packed, scaler_q, scaler_factor, scaler_mean) -> None:
        for name, whole in (("weight_nf4", packed), ("scaler_q", scaler_q), ("scaler_factor", scaler_factor)):
            mine = getattr(self, name)
            mine.copy_(whole[self.rank * mine.numel() : (self.rank + 1) * mine.numel()])
        self.scaler_mean.copy_(scaler_mean)

    @torch.no_grad()
    def quantize_(self, dense: torch.Tensor) -> None:
        """``dense`` is the whole weight (every rank passes the same values); it is coded as a whole, so the result does not depend on
        the number of ranks, and this rank's part is kept."""
        if tuple(dense.shape) != self.shape:
            raise ValueError(f"expected weight of shape {self.shape}, got {tuple(dense.shape)}")
        self._keep_own_part(*_encode(dense.to(self.weight_nf4.device), self.block_size, self.scaler_block_size))

    def _gather(self, part: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        if self.world == 1:
            return part
        if part.is_cuda:
            whole = torch.empty(self.world * part.numel(), dtype=part.dtype, device=part.device)
            dist.all_gather_into_tensor(whole, part.contiguous(), group=self.group)
            return whole
        parts = [torch.empty_like(part) for _ in range(self.world)]
        dist.all_gather(parts, part.contiguous(), group=self.group)
        return torch.cat(parts)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return _expand(self._gather(self.weight_nf4), self._gather(self.scaler_q), self._gather(self.scaler_factor), self.scaler_mean, self.shape,
                       self.block_size, self.scaler_block_size, dtype or self.dtype)

    def get_original_weight(self) -> torch.Tensor:
        return self.dequantize()

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers())


def linear_nf4(x: torch.Tensor, w: NF4Weight, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ dequant(w).T``; the weight is frozen, so autograd only needs ``dX`` and the
    dense copy is rebuilt in backward instead of being saved."""
    return _NF4Linear.apply(x, w, bias)


class _NF4Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w: NF4Weight, bias):
        from ... import ops

        ctx.w = w
        dense = w.dequantize(x.dtype)
        with torch.no_grad():
            return ops.linear(x, dense, bias)

    @staticmethod
    def backward(ctx, grad_out):
        from ... import ops

        dense = ctx.w.dequantize(grad_out.dtype)
        with torch.no_grad():
            g2 = grad_out.reshape(-1, grad_out.shape[-1])
            gx = ops.matmul(g2 if g2.is_contiguous() else g2.contiguous(), dense).view(*grad_out.shape[:-1], dense.shape[1])  # dy · W, W read in place
        gb = grad_out.reshape(-1, grad_out.shape[-1]).sum(0) if ctx.needs_input_grad[2] else None
        return gx, None, gb
