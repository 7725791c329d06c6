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
        dense = dense.to(self.weight_nf4.device)
        packed = None
        if dense.is_cuda and dense.dtype == torch.bfloat16 and self.block_size % 32 == 0:
            from ...ops import _cuda, cuda_ops_enabled

            if cuda_ops_enabled(dense):
                packed, sq, sf, mean = _cuda.nf4_quantize(dense, self.block_size, self.scaler_block_size)
        if packed is None:
            packed, sq, sf, mean = _ref.nf4_quantize(dense, self.block_size, self.scaler_block_size)
        self.weight_nf4.copy_(packed)
        self.scaler_q.copy_(sq)
        self.scaler_factor.copy_(sf)
        self.scaler_mean.copy_(mean)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        target = dtype or self.dtype
        n = self.shape[0] * self.shape[1]
        if self.weight_nf4.is_cuda and target == torch.bfloat16 and n % 16 == 0 and self.block_size % 16 == 0:
            from ...ops import _cuda, cuda_ops_enabled

            if cuda_ops_enabled(self.weight_nf4):
                return _cuda.nf4_dequantize(self.weight_nf4, self.scaler_q, self.scaler_factor, self.scaler_mean, self.shape, self.block_size, self.scaler_block_size)
        return _ref.nf4_dequantize(
            self.weight_nf4,
            self.scaler_q,
            self.scaler_factor,
            self.scaler_mean,
            self.shape,
            self.block_size,
            self.scaler_block_size,
            dtype or self.dtype,
        )

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
