"""CUDA execution path of :mod:`torchtune_b200.ops`: autograd functions over the sm_100a
kernels in ``csrc/`` (loaded through :mod:`._lib`)."""
from __future__ import annotations

import ctypes
import os
import math
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch

from . import _lib
from ._lib import check, err_word, lib, stream_ptr
from .mask import AttentionMask

_BF16 = torch.bfloat16


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ======================================================================= GEMM
_PAIR_KERNEL = os.environ.get("TTB_GEMM_2SM", "1") != "0"
_SM_PAIRS = None


def _use_pair_kernel(M: int, N: int, K: int, out: torch.Tensor) -> bool:
    """The CTA-pair kernel (``tcgen05.mma.cta_group::2``, 256 × 256 tiles, ``csrc/gemm2sm.cu``) takes bf16-output problems with
    at least one 256 × 256 tile per SM pair; smaller ones keep 128-row tiles, which spread over more SMs."""
    global _SM_PAIRS
    if not _PAIR_KERNEL or out.dtype != _BF16:
        return False
    if _SM_PAIRS is None:
        _SM_PAIRS = max(1, torch.cuda.get_device_properties(out.device).multi_processor_count // 2)
    return K >= 128 and (-(-M // 256)) * (-(-N // 256)) >= _SM_PAIRS


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = _BF16,
    accumulate: bool = False,
    bias: Optional[torch.Tensor] = None,
    alpha: float = 1.0,
) -> torch.Tensor:
    """``C[M,N] (+)= alpha * op(A) op(B)`` on the tcgen05 tensor cores.

    ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]``
    (``b_mn=False``) or ``[K,N]`` (``b_mn=True``).  Both must be bf16 with unit inner stride
    (row strides are free, multiples of 8).
    """
    assert a.dtype == _BF16 and b.dtype == _BF16 and a.dim() == 2 and b.dim() == 2
    if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
        a = a.contiguous()
    if b.stride(1) != 1 or b.stride(0) % 8 or b.data_ptr() % 16:
        b = b.contiguous()
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm contraction mismatch: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an existing `out`")
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
    if M == 0 or N == 0:
        return out
    if K == 0:
        return out if accumulate else out.zero_()
    if _use_pair_kernel(M, N, K, out):
        rc = lib().ttb_gemm_bf16_2sm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(a_mn), int(b_mn), a.stride(0), b.stride(0), out.stride(0), int(accumulate),
                                     _ptr(bias), float(alpha), err_word(a.device).data_ptr(), stream_ptr())
        check(rc, f"gemm (CTA pairs) M={M} N={N} K={K} a_mn={a_mn} b_mn={b_mn}")
        return out
    rc = lib().ttb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(a_mn), int(b_mn),
        a.stride(0), b.stride(0), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
        _ptr(bias), float(alpha), err_word(a.device).data_ptr(), stream_ptr(),
    )
    check(rc, f"gemm M={M} N={N} K={K} a_mn={a_mn} b_mn={b_mn}")
    return out


def gemm_dual(a: torch.Tensor, b: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor, *, b_mn: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a · op(b) + a2 · op(b2) (+ bias)`` in one kernel and one accumulator (the second pair extends the main loop by
    ``ceil(K2 / 64)`` k-blocks).  ``a``: ``[M, K]``, ``a2``: ``[M, K2]``; ``b``/``b2``: ``[N, K]``/``[N, K2]`` or, with ``b_mn``, ``[K, N]``/``[K2, N]``."""
    def ok(t):
        return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()

    a, b, a2, b2 = ok(a), ok(b), ok(a2), ok(b2)
    M, K = a.shape
    K2 = a2.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    out = torch.empty(M, N, dtype=_BF16, device=a.device)
    if K % 8 == 0 and K2 % 8 == 0 and _use_pair_kernel(M, N, K, out):
        rc = lib().ttb_gemm_bf16_dual_2sm(a.data_ptr(), b.data_ptr(), a2.data_ptr(), b2.data_ptr(), out.data_ptr(), M, N, K, K2, int(b_mn), a.stride(0), b.stride(0),
                                          a2.stride(0), b2.stride(0), out.stride(0), _ptr(bias), 1.0, err_word(a.device).data_ptr(), stream_ptr())
        check(rc, f"gemm_dual (CTA pairs) M={M} N={N} K={K} K2={K2} b_mn={b_mn}")
        return out
    rc = lib().ttb_gemm_bf16_dual(a.data_ptr(), b.data_ptr(), a2.data_ptr(), b2.data_ptr(), out.data_ptr(), M, N, K, K2, 0, int(b_mn), a.stride(0), b.stride(0),
                                  a2.stride(0), b2.stride(0), out.stride(0), 0, 0, _ptr(bias), 1.0, err_word(a.device).data_ptr(), stream_ptr())
    check(rc, f"gemm_dual M={M} N={N} K={K} K2={K2} b_mn={b_mn}")
    return out


def gemm_skinny(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """:func:`gemm` for outputs with so few tiles that most SMs would idle (adapter weight gradients ``[r, in]`` / ``[out, r]`` with
    a long contraction): the contraction is split over enough CTAs to fill the GPU and the partial tiles are summed in fp32."""
    def ok(t):
        return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()

    a, b = ok(a), ok(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N = b.shape[1] if b_mn else b.shape[0]
    bn = 256 if N > 128 else (128 if N > 64 else 64)
    tiles = -(-M // 128) * -(-N // bn)
    splits = min(64, 148 // tiles, -(-K // 256)) if tiles else 1
    if splits <= 1:
        return gemm(a, b, a_mn=a_mn, b_mn=b_mn, alpha=alpha)
    out = torch.zeros(M, N, dtype=torch.float32, device=a.device)
    rc = lib().ttb_gemm_bf16_splitk(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, int(a_mn), int(b_mn), a.stride(0), b.stride(0), out.stride(0), splits,
                                    float(alpha), err_word(a.device).data_ptr(), stream_ptr())
    check(rc, f"gemm_splitk M={M} N={N} K={K} splits={splits}")
    return out.to(_BF16)


def gemm_residual(a: torch.Tensor, b: torch.Tensor, residual: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M, K] · b[N, K]ᵀ (+ bias) + residual[M, N]`` with the addition in the GEMM epilogue (CTA-pair kernel); problems too small for that
    kernel run the plain GEMM followed by an add."""
    def ok(t):
        return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()

    a, b, residual = ok(a), ok(b), ok(residual)
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty(M, N, dtype=_BF16, device=a.device)
    if K % 8 == 0 and _use_pair_kernel(M, N, K, out):
        rc = lib().ttb_gemm_bf16_2sm_residual(a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), residual.stride(0),
                                              _ptr(bias), err_word(a.device).data_ptr(), stream_ptr())
        check(rc, f"gemm_residual M={M} N={N} K={K}")
        return out
    return gemm(a, b, out=out, bias=bias).add_(residual)


class _LinearResidual(torch.autograd.Function):
    """``x @ Wᵀ (+ b) + residual``: the residual gradient is the incoming gradient itself, the other two as in :class:`_Linear`."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        y = gemm_residual(x2, weight, residual.reshape(-1, weight.shape[0]), bias)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw = _wgrad(weight, dy2, x2)
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, (dy if ctx.needs_input_grad[3] else None)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], residual: torch.Tensor) -> torch.Tensor:
    return _LinearResidual.apply(x, weight, bias, residual)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        y = gemm(x2, weight, bias=bias)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw = _wgrad(weight, dy2, x2)  # dW = dYᵀ · X (possibly on the side stream)
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)  # dX = dY · W
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


def nf4_quantize(weight: torch.Tensor, block_size: int = 64, scaler_block_size: int = 256):
    """bf16 CUDA weight → ``(packed uint8, scaler_q int8, scaler_factor fp32, scaler_mean fp32)`` with the same results as
    :func:`reference.nf4_quantize`; the two passes over the weight are kernels, the coding of the per-block scales tensor ops."""
    w = weight.detach().contiguous()
    n = w.numel()
    n_blocks = n // block_size
    absmax = torch.empty(n_blocks, dtype=torch.float32, device=w.device)
    check(lib().ttb_nf4_absmax(w.data_ptr(), absmax.data_ptr(), n, block_size, stream_ptr()), "nf4_absmax")
    mean = absmax.mean()
    centred = (absmax - mean).view(-1, scaler_block_size)
    factor = 127.0 / centred.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    sq = torch.round(centred * factor).clamp(-128, 127).to(torch.int8)
    scales = ((sq.float() / factor).view(-1) + mean).contiguous()
    packed = torch.empty(n // 2, dtype=torch.uint8, device=w.device)
    check(lib().ttb_nf4_encode(w.data_ptr(), scales.data_ptr(), packed.data_ptr(), n, block_size, stream_ptr()), "nf4_encode")
    return packed, sq.view(-1), factor.view(-1).float(), mean.float()


def nf4_dequantize(packed: torch.Tensor, scaler_q: torch.Tensor, scaler_factor: torch.Tensor, scaler_mean: torch.Tensor, shape, block_size: int, scaler_block_size: int) -> torch.Tensor:
    """NF4 codes + double-quantised scales → dense bf16 ``shape`` (one streaming kernel)."""
    out = torch.empty(shape, dtype=_BF16, device=packed.device)
    mean = scaler_mean.reshape(1).to(torch.float32)
    check(lib().ttb_nf4_dequant(packed.data_ptr(), scaler_q.data_ptr(), scaler_factor.data_ptr(), mean.data_ptr(), out.data_ptr(), out.numel(), block_size, scaler_block_size, stream_ptr()), "nf4_dequant")
    return out


class _LoRALinear(torch.autograd.Function):
    """``y = x·Wᵀ (+ b) + s·(xd·Aᵀ)·Bᵀ``: the adapter product runs inside the base GEMM — its rank-r operands extend the main
    loop by one k-block and share the accumulator, so ``y`` is written once and nothing is re-read.  Backward mirrors it:
    ``dx = dy·W + (s·dy·B)·A`` in one kernel, ``dA = dtᵀ·xd``, ``dB = dyᵀ·(s·t)``.  ``xd`` is the (possibly dropped-out) adapter input."""

    @staticmethod
    def forward(ctx, x, xd, weight, bias, a, b, scale):
        shape = x.shape
        x2, xd2 = x.reshape(-1, shape[-1]), xd.reshape(-1, shape[-1])
        t = gemm(xd2, a, alpha=float(scale))  # [T, r] = s·xd·Aᵀ
        y = gemm_dual(x2, weight, t, b, bias=bias)  # base product and adapter product share one accumulator
        ctx.save_for_backward(x2, xd2, weight, a, b, t)
        ctx.scale, ctx.shape, ctx.has_bias = float(scale), shape, bias is not None
        ctx.same_input = xd.data_ptr() == x.data_ptr()
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, xd2, weight, a, b, t = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        s = ctx.scale
        dt = gemm(dy2, b, b_mn=True, alpha=s)  # [T, r] = s·dy·B
        dx = dxd = dw = db = da = dbm = None
        want_dx = ctx.needs_input_grad[0] or (ctx.same_input and ctx.needs_input_grad[1])
        if ctx.same_input:
            if want_dx:
                dx = gemm_dual(dy2, weight, dt, a, b_mn=True)  # dy·W + dt·A in one accumulator
        else:
            if want_dx:
                dx = gemm(dy2, weight, b_mn=True)
            if ctx.needs_input_grad[1]:
                dxd = gemm(dt, a, b_mn=True).view(ctx.shape)
        if ctx.needs_input_grad[2]:
            dw = _wgrad(weight, dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            db = dy2.sum(0)
        if ctx.needs_input_grad[4]:
            da = gemm_skinny(dt, xd2, a_mn=True, b_mn=True)  # [r, in]: 16 tiles, contraction over all tokens
        if ctx.needs_input_grad[5]:
            dbm = gemm_skinny(dy2, t, a_mn=True, b_mn=True)  # [out, r]; t already carries the scale
        return (dx.view(ctx.shape) if dx is not None else None), dxd, dw, db, da, dbm, None


def lora_linear(x, xd, weight, bias, a, b, scale):
    return _LoRALinear.apply(x, xd, weight, bias, a, b, scale)


class _LoRANF4Linear(torch.autograd.Function):
    """:class:`_LoRALinear` over a frozen NF4 base: the 4-bit weight is expanded to a bf16 scratch by the dequantisation kernel right
    before each of the two GEMMs that read it (forward, input gradient) and never saved — only the codes stay resident."""

    @staticmethod
    def forward(ctx, x, xd, nf4, bias, a, b, scale):
        shape = x.shape
        x2, xd2 = x.reshape(-1, shape[-1]), xd.reshape(-1, shape[-1])
        t = gemm(xd2, a, alpha=float(scale))  # [T, r] = s·xd·Aᵀ
        y = gemm_dual(x2, nf4.dequantize(_BF16), t, b, bias=bias)
        ctx.nf4, ctx.scale, ctx.shape, ctx.has_bias = nf4, float(scale), shape, bias is not None
        ctx.same_input = xd.data_ptr() == x.data_ptr()
        ctx.save_for_backward(xd2, a, b, t)
        return y.view(*shape[:-1], b.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xd2, a, b, t = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dt = gemm(dy2, b, b_mn=True, alpha=ctx.scale)  # [T, r] = s·dy·B
        dx = dxd = db = da = dbm = None
        want_dx = ctx.needs_input_grad[0] or (ctx.same_input and ctx.needs_input_grad[1])
        if ctx.same_input:
            if want_dx:
                dx = gemm_dual(dy2, ctx.nf4.dequantize(_BF16), dt, a, b_mn=True)
        else:
            if want_dx:
                dx = gemm(dy2, ctx.nf4.dequantize(_BF16), b_mn=True)
            if ctx.needs_input_grad[1]:
                dxd = gemm(dt, a, b_mn=True).view(ctx.shape)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            db = dy2.sum(0)
        if ctx.needs_input_grad[4]:
            da = gemm_skinny(dt, xd2, a_mn=True, b_mn=True)
        if ctx.needs_input_grad[5]:
            dbm = gemm_skinny(dy2, t, a_mn=True, b_mn=True)
        return (dx.view(ctx.shape) if dx is not None else None), dxd, None, db, da, dbm, None


def lora_linear_nf4(x, xd, nf4, bias, a, b, scale):
    return _LoRANF4Linear.apply(x, xd, nf4, bias, a, b, scale)


def _grouped_gemm(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """One launch over all experts: ``x`` ``[rows, K]`` sorted by expert, ``w`` ``[E, K, N]`` (``b_mn``) or ``[E, N, K]``, ``counts`` int64 ``[E]``
    on the device.  The tile → expert table is built on the device, so the call never synchronises with the host."""
    rows, K = x.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    out = torch.empty(rows, N, dtype=_BF16, device=x.device)
    max_tiles = -(-rows // 128) + E
    scratch = torch.empty(3 * max_tiles + 1, dtype=torch.int32, device=x.device)
    cnt = counts.to(torch.int64)
    cnt = cnt if cnt.is_contiguous() else cnt.contiguous()
    check(
        lib().ttb_gemm_grouped_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), cnt.data_ptr(), scratch.data_ptr(), rows, E, N, K, int(b_mn), x.stride(0), w.stride(1), w.stride(0), N,
                                    err_word(x.device).data_ptr(), stream_ptr()),
        "gemm_grouped",
    )
    return out


class _GroupedMatmul(torch.autograd.Function):
    """``y[rows of e] = x[rows of e] · w[e]`` with ``w`` ``[E, K, N]``.  Forward and the input gradient are single grouped launches;
    so is the weight gradient, whose *reduction* dimension is the ragged one (rows of the next expert that share a 64-row block are
    zeroed in shared memory before the MMAs)."""

    @staticmethod
    def forward(ctx, x, w, counts):
        ctx.save_for_backward(x, w, counts)
        return _grouped_gemm(x, w, counts, b_mn=True)

    @staticmethod
    def backward(ctx, dy):
        x, w, counts = ctx.saved_tensors
        if dy.stride(1) != 1 or dy.stride(0) % 8:
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _grouped_gemm(dy, w, counts, b_mn=False)  # per expert dy·w[e]ᵀ: w[e] read as [K_out, N_red] K-major
        if ctx.needs_input_grad[1]:
            # one launch for all experts; the ragged reduction ranges come from the device-resident counts (no host read)
            E, K, N = w.shape
            xc = x if (x.stride(1) == 1 and x.stride(0) % 8 == 0) else x.contiguous()
            owner = grad_window_owner(w)  # expert stack in a flat store: the epilogue writes its window of the flat gradient buffer
            accumulate = 0
            if owner is not None:
                out, dw = owner._grad_buffer, None
                accumulate, owner._grad_written = int(bool(owner._grad_written)), True
            else:
                out = dw = torch.empty_like(w)
            cnt = counts.to(torch.int64).contiguous()
            check(lib().ttb_gemm_grouped_wgrad_bf16(xc.data_ptr(), dy.data_ptr(), out.data_ptr(), cnt.data_ptr(), x.shape[0], E, K, N, xc.stride(0), dy.stride(0),
                                                    N, K * N, accumulate, err_word(x.device).data_ptr(), stream_ptr()), "gemm_grouped_wgrad")
        return dx, dw, None


def grouped_matmul(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    return _GroupedMatmul.apply(x, w, counts)


class _MatmulKN(torch.autograd.Function):
    """``y[T, N] = x[T, K] · w[K, N]`` with ``w`` stored reduction-dimension-major (the layout of
    grouped expert weights ``[E, K, N]``): forward reads ``w`` as an MN-major B operand, dgrad is
    the plain NT form ``dy · wᵀ`` and wgrad ``xᵀ · dy`` is the TN form."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm(x, w, b_mn=True)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        if dy.stride(1) != 1 or dy.stride(0) % 8:
            dy = dy.contiguous()
        dx = gemm(dy, w) if ctx.needs_input_grad[0] else None
        dw = gemm(x, dy, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw


def matmul_kn(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _MatmulKN.apply(x, w)


# --- weight-gradient delivery ------------------------------------------------------------
# A parameter that lives in a flat store carries `_grad_buffer` (its window of the flat
# gradient buffer).  Its weight gradient is then written (or accumulated) straight into that
# window by the GEMM epilogue and autograd receives no tensor.  Those GEMMs are issued on a
# side stream: they are independent of the dgrad chain, so the hardware fills the SMs that a
# persistent kernel's last partial wave leaves idle with tiles of the other stream's kernel.
_direct_wgrad = False
_wgrad_stream: Optional[torch.cuda.Stream] = None
_wgrad_pending = False
# data_ptr -> owning parameter.  Tensors handed to backward may be detached aliases of the
# parameter (activation checkpointing re-materialises saved tensors), so Python attributes
# cannot be relied on; the storage address of a flat-store window is stable and unique.
_grad_windows: Dict[int, torch.Tensor] = {}


def register_grad_window(param: torch.Tensor) -> None:
    _grad_windows[param.data_ptr()] = param


def unregister_grad_window(ptr: int) -> None:
    """Forget the window registered for the parameter at address ``ptr`` (its storage is being released)."""
    _grad_windows.pop(ptr, None)


def grad_window_owner(weight: torch.Tensor) -> Optional[torch.Tensor]:
    if not _direct_wgrad:
        return None
    owner = _grad_windows.get(weight.data_ptr())
    if owner is not None and owner.shape == weight.shape:
        return owner
    return None


def enable_direct_wgrad(flag: bool, use_side_stream: Optional[bool] = None) -> None:
    global _direct_wgrad, _wgrad_stream
    import os

    _direct_wgrad = flag
    if use_side_stream is None:
        use_side_stream = os.environ.get("TTB_WGRAD_STREAM", "1") != "0"
    _wgrad_stream = torch.cuda.Stream() if (flag and use_side_stream) else None


def join_wgrad_stream() -> None:
    """Make the current stream wait for every weight-gradient GEMM issued so far."""
    global _wgrad_pending
    if _wgrad_stream is not None and _wgrad_pending:
        torch.cuda.current_stream().wait_stream(_wgrad_stream)
        _wgrad_pending = False


def _wgrad(weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    global _wgrad_pending
    owner = grad_window_owner(weight)
    if owner is None:
        return gemm(dy2, x2, a_mn=True, b_mn=True)
    buf = owner._grad_buffer
    accumulate = bool(owner._grad_written)
    owner._grad_written = True
    if _wgrad_stream is None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=buf, accumulate=accumulate)
        return None
    cur = torch.cuda.current_stream()
    _wgrad_stream.wait_stream(cur)
    with torch.cuda.stream(_wgrad_stream):
        gemm(dy2, x2, a_mn=True, b_mn=True, out=buf, accumulate=accumulate)
    dy2.record_stream(_wgrad_stream)
    x2.record_stream(_wgrad_stream)
    _wgrad_pending = True
    return None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    K, N = x.shape[-1], weight.shape[0]
    if K % 8 or N % 8:  # TMA needs 16-byte row pitches; odd sizes (tiny classifier heads) use the library path
        return torch.nn.functional.linear(x, weight, bias)
    return _Linear.apply(x, weight, bias)


# ======================================================================= embedding
class _Embedding(torch.autograd.Function):
    """Row gather; the gradient sorts the ids and sums every run of equal ids in fp32 (deterministic, no atomics).
    A table that owns a window of a flat gradient buffer receives its gradient there and autograd gets no tensor."""

    @staticmethod
    def forward(ctx, ids, table, padding_idx):
        flat = ids.reshape(-1)
        if flat.dtype != torch.int64:
            flat = flat.long()
        flat = flat.contiguous()
        n, (vocab, dim) = flat.numel(), table.shape
        out = torch.empty(n, dim, dtype=table.dtype, device=table.device)
        check(lib().ttb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), n, dim, vocab, stream_ptr()), "embedding_fwd")
        ctx.save_for_backward(flat, table)
        ctx.padding_idx = -1 if padding_idx is None else int(padding_idx)
        return out.view(*ids.shape, dim)

    @staticmethod
    def backward(ctx, dy):
        flat, table = ctx.saved_tensors
        vocab, dim = table.shape
        dy2 = dy.reshape(-1, dim)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        sorted_ids, order = torch.sort(flat, stable=True)
        owner = grad_window_owner(table)
        if owner is None:
            dtable = torch.zeros_like(table)
        else:
            dtable = owner._grad_buffer
            join_wgrad_stream()  # a tied output projection writes the same window from the side stream
            if not owner._grad_written:
                dtable.zero_()
            owner._grad_written = True
        check(lib().ttb_embedding_bwd(sorted_ids.data_ptr(), order.data_ptr(), dy2.data_ptr(), dtable.data_ptr(), flat.numel(), dim, vocab, ctx.padding_idx, stream_ptr()), "embedding_bwd")
        return None, (dtable if owner is None else None), None


def embedding(ids: torch.Tensor, table: torch.Tensor, padding_idx: Optional[int] = None) -> torch.Tensor:
    return _Embedding.apply(ids, table, padding_idx)


def moe_route_sort(expert_ids: torch.Tensor, num_experts: int, with_inverse: bool = False):
    """Stable counting sort of routed pairs by expert: ``(counts [E], order [n])`` (+ ``inverse [n]``: where each pair went)."""
    ids = expert_ids.to(torch.int64).contiguous()
    n = ids.numel()
    counts = torch.empty(num_experts, dtype=torch.int64, device=ids.device)
    order = torch.empty(n, dtype=torch.int64, device=ids.device)
    inverse = torch.empty(n, dtype=torch.int64, device=ids.device) if with_inverse else None
    L = lib()
    L.ttb_moe_route_sort.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    check(L.ttb_moe_route_sort(ids.data_ptr(), n, num_experts, counts.data_ptr(), order.data_ptr(), _ptr(inverse), stream_ptr()), "moe_route_sort")
    return (counts, order, inverse) if with_inverse else (counts, order)


def _declare_route(L) -> None:
    if getattr(L, "_route_declared", False):
        return
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    L.ttb_moe_route.argtypes = [vp, i32, i64, i32, i32, vp, vp, vp]
    L.ttb_moe_route_bwd.argtypes = [vp, i32, vp, vp, i64, i32, i32, vp, vp]
    L.ttb_moe_gather_rows.argtypes = [vp, vp, vp, vp, i64, i32, i64, vp]
    L.ttb_moe_combine_rows.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, i64, vp]
    L.ttb_moe_row_dots.argtypes = [vp, vp, vp, vp, i64, i32, i64, vp]
    for fn in (L.ttb_moe_route, L.ttb_moe_route_bwd, L.ttb_moe_gather_rows, L.ttb_moe_combine_rows, L.ttb_moe_row_dots):
        fn.restype = i32
    L._route_declared = True


class _MoERoute(torch.autograd.Function):
    """Gate logits ``[T, E]`` → ``(scores [T, k] bf16, selected [T, k] int64)``: sigmoid and top-k in one kernel, one warp per token."""

    @staticmethod
    def forward(ctx, logits, k):
        T, E = logits.shape
        L = lib()
        _declare_route(L)
        lg = logits.contiguous()
        scores = torch.empty(T, k, dtype=_BF16, device=lg.device)
        selected = torch.empty(T, k, dtype=torch.int64, device=lg.device)
        check(L.ttb_moe_route(lg.data_ptr(), int(lg.dtype == torch.float32), T, E, k, scores.data_ptr(), selected.data_ptr(), stream_ptr()), "moe_route")
        ctx.save_for_backward(lg, selected)
        ctx.k = k
        ctx.mark_non_differentiable(selected)
        return scores, selected

    @staticmethod
    def backward(ctx, dscores, _dsel):
        lg, selected = ctx.saved_tensors
        T, E = lg.shape
        dl = torch.empty_like(lg)
        check(lib().ttb_moe_route_bwd(lg.data_ptr(), int(lg.dtype == torch.float32), selected.data_ptr(), dscores.to(_BF16).contiguous().data_ptr(), T, E, ctx.k, dl.data_ptr(), stream_ptr()),
              "moe_route_bwd")
        return dl, None


def moe_route(logits: torch.Tensor, k: int):
    return _MoERoute.apply(logits, k)


def _gather_rows(x, idx, scale):
    P, D = idx.numel(), x.shape[1]
    out = torch.empty(P, D, dtype=_BF16, device=x.device)
    if P:
        check(lib().ttb_moe_gather_rows(x.data_ptr(), idx.data_ptr(), _ptr(scale), out.data_ptr(), P, D, x.shape[0], stream_ptr()), "moe_gather_rows")
    return out


def _combine_rows(src, inv, scale, base, T, k):
    D = src.shape[1]
    out = torch.empty(T, D, dtype=_BF16, device=src.device)
    check(lib().ttb_moe_combine_rows(src.data_ptr(), inv.data_ptr(), _ptr(scale), _ptr(base), out.data_ptr(), T, k, D, src.shape[0], stream_ptr()), "moe_combine_rows")
    return out


class _MoEGather(torch.autograd.Function):
    """``out[j] = x[idx[j]] · scale[j]`` for the pairs in expert order; ``inv [T·k]`` is the position of pair (t, s) in that order,
    which turns the gradient with respect to ``x`` into a pull (no atomics)."""

    @staticmethod
    def forward(ctx, x, idx, scale, inv, k):
        _declare_route(lib())
        x, idx, inv = x.contiguous(), idx.contiguous(), inv.contiguous()
        scale = None if scale is None else scale.to(_BF16).contiguous()
        ctx.save_for_backward(x, idx, scale, inv)
        ctx.k = k
        return _gather_rows(x, idx, scale)

    @staticmethod
    def backward(ctx, dout):
        x, idx, scale, inv = ctx.saved_tensors
        dout = dout.contiguous()
        dx = dscale = None
        if ctx.needs_input_grad[0]:
            dx = _combine_rows(dout, inv, scale, None, x.shape[0], ctx.k)
        if scale is not None and ctx.needs_input_grad[2]:
            dscale = torch.empty(idx.numel(), dtype=_BF16, device=x.device)
            if idx.numel():
                check(lib().ttb_moe_row_dots(x.data_ptr(), idx.data_ptr(), dout.data_ptr(), dscale.data_ptr(), idx.numel(), x.shape[1], x.shape[0], stream_ptr()), "moe_row_dots")
        return dx, None, dscale, None, None


class _MoECombine(torch.autograd.Function):
    """``out[t] = base[t] + Σ_s src[inv[t·k + s]]`` — the expert outputs back in token order, summed over the token's experts."""

    @staticmethod
    def forward(ctx, src, inv, idx, base, k):
        _declare_route(lib())
        src, inv, idx = src.contiguous(), inv.contiguous(), idx.contiguous()
        base = None if base is None else base.contiguous()
        T = inv.numel() // k
        ctx.save_for_backward(idx)
        ctx.rows = src.shape[0]
        ctx.has_base = base is not None
        return _combine_rows(src, inv, None, base, T, k)

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dout = dout.contiguous()
        dsrc = None
        if ctx.needs_input_grad[0]:
            g = _gather_rows(dout, idx, None)
            dsrc = g if g.shape[0] == ctx.rows else torch.cat([g, g.new_zeros(ctx.rows - g.shape[0], g.shape[1])])
        return dsrc, None, None, (dout if ctx.has_base and ctx.needs_input_grad[3] else None), None


def moe_gather(x, idx, scale, inv, k):
    return _MoEGather.apply(x, idx, scale, inv, k)


def moe_combine(src, inv, idx, base, k):
    return _MoECombine.apply(src, inv, idx, base, k)


def moe_permute_indices(tokens_per_expert_group: torch.Tensor, experts_per_rank: int, num_ranks: int, max_len: int, alignment: int):
    counts = tokens_per_expert_group.reshape(-1).to(torch.int64).contiguous()
    dev = counts.device
    permuted = torch.empty(max_len, dtype=torch.int32, device=dev)
    m_sizes = torch.empty(experts_per_rank, dtype=torch.int32, device=dev)
    m_offsets = torch.empty(experts_per_rank, dtype=torch.int32, device=dev)
    check(lib().ttb_moe_permute_indices(counts.data_ptr(), experts_per_rank, num_ranks, max_len, alignment, permuted.data_ptr(), m_sizes.data_ptr(), m_offsets.data_ptr(), stream_ptr()), "moe_permute_indices")
    return permuted, m_sizes, m_offsets


# ======================================================================= fp8 linear
_FP8_MAX = {False: 448.0, True: 57344.0}  # e4m3, e5m2


def fp8_scales(x2: torch.Tensor, e5m2: bool, rowwise: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantisation scales ``fmax / amax`` for the two layouts of ``x2`` ``[R, C]``: per row (for the same-layout copy) and per
    column (for the transposed copy); with tensorwise scaling both are the same single value."""
    fmax = _FP8_MAX[e5m2]
    if rowwise:
        a = x2.abs()
        return fmax / a.amax(dim=1).float().clamp_min(1e-12), fmax / a.amax(dim=0).float().clamp_min(1e-12)
    s = (fmax / x2.abs().amax().float().clamp_min(1e-12)).reshape(1)
    return s, s


def fp8_cast(x2: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor, *, e5m2: bool = False, want: bool = True, want_t: bool = True):
    """``(fp8(x2 · s_row), fp8(x2 · s_col)ᵀ)`` as uint8 tensors ``[R, C]`` / ``[C, R]`` in one pass over ``x2`` (bf16)."""
    R, C = x2.shape
    out = torch.empty(R, C, dtype=torch.uint8, device=x2.device) if want else None
    out_t = torch.empty(C, R, dtype=torch.uint8, device=x2.device) if want_t else None
    check(lib().ttb_fp8_cast_transpose(x2.data_ptr(), x2.stride(0), R, C, s_row.data_ptr(), int(s_row.numel() > 1), _ptr(out), s_col.data_ptr(), int(s_col.numel() > 1),
                                       _ptr(out_t), int(e5m2), stream_ptr()), "fp8_cast_transpose")
    return out, out_t


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, inv_sa: torch.Tensor, inv_sb: torch.Tensor, *, a_e5m2: bool = False, b_e5m2: bool = False,
             bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``(a[M, K] · b[N, K]ᵀ) · inv_sa[m] · inv_sb[n] (+ bias)`` → bf16 ``[M, N]``; ``a``, ``b`` uint8-stored fp8."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    check(lib().ttb_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), int(a_e5m2), int(b_e5m2),
                             inv_sa.data_ptr(), int(inv_sa.numel() > 1), inv_sb.data_ptr(), int(inv_sb.numel() > 1), _ptr(bias), int(accumulate),
                             err_word(a.device).data_ptr(), stream_ptr()), "gemm_fp8")
    return out


class _Fp8Linear(torch.autograd.Function):
    """``x @ Wᵀ (+ bias)`` with all three products (forward, input gradient, weight gradient) on the fp8 tensor cores.  Inputs are
    quantised dynamically (tensorwise: e4m3 activations / weights, e5m2 output gradients; rowwise: e4m3 with one scale per row of
    each operand along its contraction dimension).  Only fp8 copies are saved for backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, rowwise: bool):
        K, N = x.shape[-1], weight.shape[0]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        sx_row, sx_col = fp8_scales(x2, False, rowwise)
        sw_row, sw_col = fp8_scales(weight, False, rowwise)
        need_dw, need_dx = weight.requires_grad, x.requires_grad
        xq, xq_t = fp8_cast(x2, sx_row, sx_col, want_t=need_dw)
        wq, wq_t = fp8_cast(weight, sw_row, sw_col, want_t=need_dx)
        y = gemm_fp8(xq, wq, 1.0 / sx_row, 1.0 / sw_row, bias=bias)
        ctx.rowwise, ctx.has_bias = rowwise, bias is not None
        ctx.save_for_backward(xq_t, None if xq_t is None else 1.0 / sx_col, wq_t, None if wq_t is None else 1.0 / sw_col, weight)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        xq_t, inv_sx_col, wq_t, inv_sw_col, weight = ctx.saved_tensors
        N = dy.shape[-1]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        e5m2 = not ctx.rowwise
        s_row, s_col = fp8_scales(dy2, e5m2, ctx.rowwise)
        dyq, dyq_t = fp8_cast(dy2, s_row, s_col, e5m2=e5m2, want=wq_t is not None, want_t=xq_t is not None)
        dx = dw = db = None
        if wq_t is not None:
            dx = gemm_fp8(dyq, wq_t, 1.0 / s_row, inv_sw_col, a_e5m2=e5m2).view(*dy.shape[:-1], wq_t.shape[0])
        if xq_t is not None:
            owner = grad_window_owner(weight)
            if owner is None:
                dw = gemm_fp8(dyq_t, xq_t, 1.0 / s_col, inv_sx_col, a_e5m2=e5m2)
            else:
                gemm_fp8(dyq_t, xq_t, 1.0 / s_col, inv_sx_col, a_e5m2=e5m2, out=owner._grad_buffer, accumulate=bool(owner._grad_written))
                owner._grad_written = True
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, rowwise: bool = False) -> torch.Tensor:
    return _Fp8Linear.apply(x, weight, bias, rowwise)


# ======================================================================= block-scaled (MX) fp8 linear
def mx_quantize(x2: torch.Tensor, transpose: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 values (uint8 storage) and the packed scale buffer of a bf16 ``[R, C]`` operand, blocks of 32 along ``C``; with
    ``transpose`` the operand is ``x2.T`` (``[C, R]``, blocks along ``R``).  Scale buffer layout: gemm_mxfp8.cu."""
    assert x2.dim() == 2 and x2.dtype == _BF16 and x2.stride(1) == 1
    R, C = x2.shape
    rows, k = (C, R) if transpose else (R, C)
    q = torch.empty(rows, k, dtype=torch.uint8, device=x2.device)
    sf = torch.zeros(lib().ttb_mx_scale_bytes(rows, k), dtype=torch.uint8, device=x2.device)
    check(lib().ttb_mx_quantize(x2.data_ptr(), x2.stride(0), q.data_ptr(), q.stride(0), sf.data_ptr(), R, C, int(transpose), stream_ptr()), f"mx_quantize {R}x{C} transpose={transpose}")
    return q, sf


def mx_quantize_both(x2: torch.Tensor) -> Tuple[Tuple[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]:
    """``(mx_quantize(x2), mx_quantize(x2, transpose=True))`` from one pass over ``x2`` (both dimensions multiples of 32)."""
    assert x2.dim() == 2 and x2.dtype == _BF16 and x2.stride(1) == 1
    R, C = x2.shape
    q = torch.empty(R, C, dtype=torch.uint8, device=x2.device)
    qt = torch.empty(C, R, dtype=torch.uint8, device=x2.device)
    sf = torch.zeros(lib().ttb_mx_scale_bytes(R, C), dtype=torch.uint8, device=x2.device)
    sft = torch.zeros(lib().ttb_mx_scale_bytes(C, R), dtype=torch.uint8, device=x2.device)
    check(lib().ttb_mx_quantize_both(x2.data_ptr(), x2.stride(0), q.data_ptr(), q.stride(0), sf.data_ptr(), qt.data_ptr(), qt.stride(0), sft.data_ptr(), R, C, stream_ptr()),
          f"mx_quantize_both {R}x{C}")
    return (q, sf), (qt, sft)


def mx_unpack_scales(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """``[rows, k / 32]`` exponent bytes read back from the packed scale buffer (tests and debugging)."""
    r = torch.arange(rows, device=sf.device).unsqueeze(1)
    b = torch.arange(k // 32, device=sf.device).unsqueeze(0)
    chunks_per_row = (k + 127) // 128
    off = ((r >> 7) * chunks_per_row + (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)
    return sf[off]


def gemm_mxfp8(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor, *, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               accumulate: bool = False) -> torch.Tensor:
    """``aq[M, K] · bq[N, K]ᵀ`` with per-32 block scales applied by the tensor core (+ bias) → bf16 ``[M, N]``."""
    M, K = aq.shape
    N = bq.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=_BF16, device=aq.device)
    check(lib().ttb_gemm_mxfp8(aq.data_ptr(), bq.data_ptr(), asf.data_ptr(), bsf.data_ptr(), out.data_ptr(), M, N, K, aq.stride(0), bq.stride(0), out.stride(0), _ptr(bias),
                               int(accumulate), err_word(aq.device).data_ptr(), stream_ptr()), f"gemm_mxfp8 M={M} N={N} K={K}")
    return out


# The most recent activation quantised in each orientation.  Projections that read the same tensor (q / k / v, gate / up) hit it
# instead of quantising again; the entry keeps that tensor alive, so its address cannot be handed to another tensor meanwhile,
# and the version counter catches in-place changes.
_MX_LAST: dict = {}


def _mx_quantize_shared(x2: torch.Tensor, transpose: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    ent = _MX_LAST.get(transpose)
    if ent is not None:
        t, version, q, sf = ent
        if t.data_ptr() == x2.data_ptr() and t.shape == x2.shape and t.stride() == x2.stride() and version == x2._version and t.device == x2.device:
            return q, sf
    q, sf = mx_quantize(x2, transpose)
    _MX_LAST[transpose] = (x2, x2._version, q, sf)
    return q, sf


def _mx_entry(x2: torch.Tensor, transpose: bool):
    ent = _MX_LAST.get(transpose)
    if ent is not None:
        t, version, q, sf = ent
        if t.data_ptr() == x2.data_ptr() and t.shape == x2.shape and t.stride() == x2.stride() and version == x2._version and t.device == x2.device:
            return q, sf
    return None


def _mx_quantize_shared_pair(x2: torch.Tensor):
    """Both orientations of an activation; one fused pass when neither is in the shared entries yet."""
    plain, transposed = _mx_entry(x2, False), _mx_entry(x2, True)
    if plain is None and transposed is None and x2.shape[0] % 32 == 0 and x2.shape[1] % 32 == 0:
        plain, transposed = mx_quantize_both(x2)
        _MX_LAST[False] = (x2, x2._version, *plain)
        _MX_LAST[True] = (x2, x2._version, *transposed)
        return plain, transposed
    return (plain or _mx_quantize_shared(x2, False)), (transposed or _mx_quantize_shared(x2, True))


def mx_clear_shared() -> None:
    _MX_LAST.clear()


class _MXFp8Linear(torch.autograd.Function):
    """``x @ Wᵀ (+ bias)`` with forward, input-gradient and weight-gradient products on the block-scaled fp8 tensor-core path.  Every
    operand is quantised along its own contraction dimension (six quantisations per layer and step); only fp8 copies and their
    scales are kept for backward."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        K, N = x.shape[-1], weight.shape[0]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        need_dw, need_dx = weight.requires_grad, x.requires_grad
        if need_dw:
            (xq, xs), xt = _mx_quantize_shared_pair(x2)  # xt: [K, T], blocks along tokens
        else:
            (xq, xs), xt = _mx_quantize_shared(x2, False), (None, None)
        wq, ws = mx_quantize(weight)
        y = gemm_mxfp8(xq, xs, wq, ws, bias=bias)
        wt = mx_quantize(weight, transpose=True) if need_dx else (None, None)  # [K, N], blocks along N
        ctx.has_bias = bias is not None
        ctx.save_for_backward(xt[0], xt[1], wt[0], wt[1], weight)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        xtq, xts, wtq, wts, weight = ctx.saved_tensors
        N = dy.shape[-1]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        both = wtq is not None and xtq is not None and dy2.shape[0] % 32 == 0 and dy2.shape[1] % 32 == 0
        if both:
            (dyq, dys), (dytq, dyts) = mx_quantize_both(dy2)
        if wtq is not None:
            if not both:
                dyq, dys = mx_quantize(dy2)  # blocks along N
            dx = gemm_mxfp8(dyq, dys, wtq, wts).view(*dy.shape[:-1], wtq.shape[0])
        if xtq is not None:
            if not both:
                dytq, dyts = mx_quantize(dy2, transpose=True)  # [N, T], blocks along tokens
            owner = grad_window_owner(weight)
            if owner is None:
                dw = gemm_mxfp8(dytq, dyts, xtq, xts)
            else:
                gemm_mxfp8(dytq, dyts, xtq, xts, out=owner._grad_buffer, accumulate=bool(owner._grad_written))
                owner._grad_written = True
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


def mxfp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _MXFp8Linear.apply(x, weight, bias)


# ======================================================================= RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        check(lib().ttb_rmsnorm_fwd(x2.data_ptr(), _ptr(scale), y.data_ptr(), rstd.data_ptr(), rows, D, float(eps), stream_ptr()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, scale, rstd)
        ctx.has_scale = scale is not None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, scale, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        partial = None
        if ctx.has_scale and ctx.needs_input_grad[1]:
            n_part = lib().ttb_rmsnorm_bwd_partials(rows)
            partial = torch.empty(n_part, D, dtype=torch.float32, device=x2.device)
        check(lib().ttb_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), _ptr(scale), rstd.data_ptr(), dx.data_ptr(), _ptr(partial), rows, D, stream_ptr()), "rmsnorm_bwd")
        dscale = partial.sum(0).to(scale.dtype) if partial is not None else None
        return dx.view(dy.shape), dscale, None


def rms_norm(x: torch.Tensor, scale: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    if x.dtype != _BF16 or x.shape[-1] % 8 or x.shape[-1] > 16384 or (scale is not None and scale.dtype != _BF16):
        from . import reference

        return reference.rms_norm(x, scale, eps)
    return _RMSNorm.apply(x, scale, eps)


# ======================================================================= log-probabilities of given tokens from logits
class _LogitsLogprobs(torch.autograd.Function):
    """``log_softmax(logits / T)[token]`` per row through the cross-entropy kernel: the only [rows, V] tensor is one bf16 copy of the
    scaled logits, which the kernel overwrites with ``softmax − onehot`` for the backward pass."""

    @staticmethod
    def forward(ctx, logits2d, tokens, temperature: float):
        rows, V = logits2d.shape
        need_grad = logits2d.requires_grad
        scaled = (logits2d / temperature) if temperature != 1.0 else (logits2d.clone() if need_grad else logits2d)
        if not scaled.is_contiguous():
            scaled = scaled.contiguous()
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
        check(lib().ttb_softmax_ce(scaled.data_ptr(), tokens.data_ptr(), loss_rows.data_ptr(), None, rows, V, scaled.stride(0), -(1 << 62), 0 if need_grad else 1, stream_ptr()),
              "softmax_ce (log-probabilities)")
        ctx.temperature = temperature
        ctx.save_for_backward(scaled if need_grad else None)
        return -loss_rows

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        if grad is None:
            return None, None, None
        return grad * (-g / ctx.temperature).to(grad.dtype).unsqueeze(-1), None, None


def logits_logprobs(logits: torch.Tensor, tokens: torch.Tensor, temperature: float) -> torch.Tensor:
    V = logits.shape[-1]
    out = _LogitsLogprobs.apply(logits.reshape(-1, V), tokens.reshape(-1).contiguous(), float(temperature))
    return out.view(tokens.shape)


# ======================================================================= sampling
def sample(logits: torch.Tensor, q: torch.Tensor, temperature: float, top_k: Optional[int]) -> torch.Tensor:
    """One token per row of ``logits`` (``[rows, V]``, bf16 or fp32): temperature, optional top-k and the exponential-race draw
    ``argmax(softmax(logits / T) / q)`` in one kernel; ``q``: fp32 ``[rows, V]`` draws from Exp(1).  Returns int32 ``[rows]``."""
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib().ttb_sample(logits.data_ptr(), logits.stride(0), int(logits.dtype == _BF16), q.data_ptr(), q.stride(0), out.data_ptr(), rows, V, float(temperature),
                           int(top_k or 0), stream_ptr()), "sample")
    return out


# ======================================================================= distillation divergences
class _KDDivergence(torch.autograd.Function):
    """Sum over rows of ``w_fwd · (−Σ p_t log p_s) + w_rev · Σ p_s (log p_s − log p_t)`` for bf16 ``[rows, V]`` student / teacher logits;
    rows whose label equals ``ignore_index`` are skipped.  The gradient with respect to the student logits is produced by the same
    kernel launch (bf16), so neither softmax is ever materialised in fp32."""

    @staticmethod
    def forward(ctx, student, teacher, labels, w_fwd: float, w_rev: float, ignore_index: int):
        rows, V = student.shape
        loss_rows = torch.empty(rows, dtype=torch.float32, device=student.device)
        grad = torch.empty_like(student) if student.requires_grad else None
        check(lib().ttb_kd_divergence(student.data_ptr(), teacher.data_ptr(), labels.data_ptr(), loss_rows.data_ptr(), _ptr(grad), rows, V, student.stride(0), teacher.stride(0),
                                      grad.stride(0) if grad is not None else 0, int(ignore_index), float(w_fwd), float(w_rev), stream_ptr()), "kd_divergence")
        ctx.save_for_backward(grad)
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad * g.to(grad.dtype)) if grad is not None else None, None, None, None, None, None


def kd_divergence(student: torch.Tensor, teacher: torch.Tensor, labels: torch.Tensor, w_fwd: float, w_rev: float, ignore_index: int) -> torch.Tensor:
    def rows2d(t):
        t = t.reshape(-1, t.shape[-1])
        return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()

    return _KDDivergence.apply(rows2d(student), rows2d(teacher.detach()), labels.reshape(-1).contiguous(), w_fwd, w_rev, ignore_index)


# ======================================================================= RoPE
def _rope_launch(x: torch.Tensor, cache: torch.Tensor, pos: Optional[torch.Tensor], interleaved: bool, inverse: bool) -> torch.Tensor:
    b, s, h, d = x.shape
    if not x.is_contiguous():
        x = x.contiguous()
    y = torch.empty_like(x)
    check(lib().ttb_rope(x.data_ptr(), y.data_ptr(), cache.data_ptr(), _ptr(pos), b * s, h, d, s, int(interleaved), int(inverse), int(cache.shape[0]), stream_ptr()), "rope")
    return y


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cache, pos, interleaved):
        ctx.save_for_backward(cache, pos)
        ctx.interleaved = interleaved
        return _rope_launch(x, cache, pos, interleaved, False)

    @staticmethod
    def backward(ctx, dy):
        cache, pos = ctx.saved_tensors
        # a rotation is orthogonal: its transpose is the rotation by the negative angle
        return _rope_launch(dy, cache, pos, ctx.interleaved, True), None, None, None


def rope(x: torch.Tensor, cache: torch.Tensor, input_pos: Optional[torch.Tensor], interleaved: bool) -> torch.Tensor:
    b, s, h, d = x.shape
    if d % 16 or cache.dtype != torch.float32 or not cache.is_contiguous():
        from . import reference

        return (reference.rope_interleaved if interleaved else reference.rope_half)(x, cache, input_pos)
    pos = None
    if input_pos is not None:
        pos = input_pos.to(device=x.device, dtype=torch.int32)
        pos = pos.expand(b, s).contiguous() if pos.dim() == 2 else pos.view(1, s).expand(b, s).contiguous()
    return _RoPE.apply(x, cache, pos, interleaved)


# ======================================================================= SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        H = gate.shape[-1]
        g2, u2 = gate.reshape(-1, H), up.reshape(-1, H)
        if g2.stride(1) != 1:
            g2 = g2.contiguous()
        if u2.stride(1) != 1:
            u2 = u2.contiguous()
        y = torch.empty(g2.shape, dtype=gate.dtype, device=gate.device)
        check(lib().ttb_swiglu_fwd(g2.data_ptr(), u2.data_ptr(), y.data_ptr(), g2.shape[0], H, g2.stride(0), u2.stride(0), y.stride(0), stream_ptr()), "swiglu_fwd")
        ctx.save_for_backward(g2, u2)
        return y.view(gate.shape)

    @staticmethod
    def backward(ctx, dy):
        g2, u2 = ctx.saved_tensors
        rows, H = g2.shape
        dy2 = dy.reshape(rows, H)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dg = torch.empty(rows, H, dtype=g2.dtype, device=g2.device)
        du = torch.empty(rows, H, dtype=g2.dtype, device=g2.device)
        check(lib().ttb_swiglu_bwd(dy2.data_ptr(), g2.data_ptr(), u2.data_ptr(), dg.data_ptr(), du.data_ptr(), rows, H, dy2.stride(0), g2.stride(0), u2.stride(0), H, H, stream_ptr()), "swiglu_bwd")
        return dg.view(dy.shape), du.view(dy.shape)


class _GateUpSwiGLU(torch.autograd.Function):
    """``silu(x · W1ᵀ) ⊙ (x · W3ᵀ)`` as one launch of the CTA-pair GEMM: the even CTA of a pair loads rows of ``W1``, the odd one the same
    rows of ``W3``, and the epilogue applies the activation (``csrc/gemm2sm.cu``, SWIGLU form).  In a gradient-free pass (the first forward
    under activation checkpointing) the two pre-activations never reach HBM; otherwise the epilogue also stores them for backward, which
    is the existing SwiGLU-backward kernel followed by the usual input- and weight-gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, w1, w3):
        K, N = x.shape[-1], w1.shape[0]
        x2 = x.reshape(-1, K)
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        M = x2.shape[0]
        keep = any(ctx.needs_input_grad)
        h = torch.empty(M, N, dtype=_BF16, device=x.device)
        g = torch.empty(M, N, dtype=_BF16, device=x.device) if keep else None
        u = torch.empty(M, N, dtype=_BF16, device=x.device) if keep else None
        L = lib()
        if not getattr(L, "_swiglu_gemm_declared", False):
            vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
            L.ttb_gemm_swiglu_bf16_2sm.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, vp, vp]
            L.ttb_gemm_swiglu_bf16_2sm.restype = i32
            L._swiglu_gemm_declared = True
        check(L.ttb_gemm_swiglu_bf16_2sm(x2.data_ptr(), w1.data_ptr(), w3.data_ptr(), h.data_ptr(), _ptr(g), _ptr(u), M, N, K, x2.stride(0), w1.stride(0), N,
                                         err_word(x.device).data_ptr(), stream_ptr()), f"gate/up GEMM + SwiGLU M={M} N={N} K={K}")
        ctx.save_for_backward(x2, w1, w3, g, u)
        ctx.x_shape = x.shape
        return h.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dh):
        x2, w1, w3, g, u = ctx.saved_tensors
        M, N = g.shape
        dh2 = dh.reshape(M, N)
        if dh2.stride(1) != 1:
            dh2 = dh2.contiguous()
        dg = torch.empty(M, N, dtype=_BF16, device=g.device)
        du = torch.empty(M, N, dtype=_BF16, device=g.device)
        check(lib().ttb_swiglu_bwd(dh2.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(), M, N, dh2.stride(0), N, N, N, N, stream_ptr()), "swiglu_bwd")
        dx = dw1 = dw3 = None
        if ctx.needs_input_grad[1]:
            dw1 = _wgrad(w1, dg, x2)
        if ctx.needs_input_grad[2]:
            dw3 = _wgrad(w3, du, x2)
        if ctx.needs_input_grad[0]:
            dx = gemm(dg, w1, b_mn=True)
            gemm(du, w3, b_mn=True, out=dx, accumulate=True)
            dx = dx.view(ctx.x_shape)
        return dx, dw1, dw3


def gate_up_swiglu(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor) -> Optional[torch.Tensor]:
    """Fused gate / up projections + SwiGLU, or ``None`` when the shapes do not suit the CTA-pair kernel (the caller then runs the three
    separate operators)."""
    if not _PAIR_KERNEL or os.environ.get("TTB_FUSE_SWIGLU", "1") == "0":
        return None
    K, N = x.shape[-1], w1.shape[0]
    M = x.numel() // K
    if w1.shape != w3.shape or w1.dtype != _BF16 or w3.dtype != _BF16 or K % 8 or N % 8 or not (w1.is_contiguous() and w3.is_contiguous()):
        return None
    if w1.data_ptr() % 16 or w3.data_ptr() % 16:
        return None
    global _SM_PAIRS
    if _SM_PAIRS is None:
        _SM_PAIRS = max(1, torch.cuda.get_device_properties(x.device).multi_processor_count // 2)
    if K < 128 or (-(-M // 256)) * (-(-N // 128)) < _SM_PAIRS:
        return None
    return _GateUpSwiGLU.apply(x, w1, w3)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape[-1] % 8:
        from . import reference

        return reference.swiglu(gate, up)
    return _SwiGLU.apply(gate, up)


# ======================================================================= attention
def attention(q, k, v, mask: AttentionMask, scale: Optional[float], softcap: float) -> torch.Tensor:
    from ._cuda_attention import attention as _attn

    return _attn(q, k, v, mask, scale, softcap)


# ======================================================================= fused linear + CE
def _ce_chunk_rows(T: int, num_chunks: int) -> int:
    return max(1, -(-T // max(1, num_chunks)))


# Above this many bytes of bf16 logits the token dimension is processed in chunks; below it the
# whole batch is one pass (one logits GEMM, one dgrad, one wgrad written once in bf16).
_CE_SINGLE_PASS_BYTES = 6 * 2**30


class _LinearCE(torch.autograd.Function):
    """Loss and both gradients in one forward sweep: logits = H·Wᵀ (bf16, as the unfused bf16
    projection produces), softmax-CE turns them into dlogits in place, then dH = dlogits·W and
    dW = dlogitsᵀ·H while the logits are still hot.  ``num_chunks`` bounds memory: chunking is
    only used when the full logits buffer would exceed ``_CE_SINGLE_PASS_BYTES``."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, num_chunks, softcap=0.0):
        D = hidden.shape[-1]
        h2 = hidden.reshape(-1, D)
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        y = labels.reshape(-1).to(torch.int64).contiguous()
        T, V = h2.shape[0], weight.shape[0]
        need_h = ctx.needs_input_grad[0]
        need_w = ctx.needs_input_grad[1]
        if T * V * 2 <= _CE_SINGLE_PASS_BYTES:
            num_chunks = 1
        rows = _ce_chunk_rows(T, num_chunks)
        single = rows >= T
        loss_rows = torch.empty(T, dtype=torch.float32, device=h2.device)
        dh = torch.empty_like(h2) if need_h else None
        owner = grad_window_owner(weight) if (need_w and single) else None
        direct = owner is not None
        dw = None
        if need_w and not direct:
            dw = torch.empty(V, D, dtype=_BF16, device=h2.device) if single else torch.zeros(V, D, dtype=torch.float32, device=h2.device)
        buf = torch.empty(min(rows, T), V, dtype=_BF16, device=h2.device)
        L = lib()
        for start in range(0, T, rows):
            n = min(rows, T - start)
            hc = h2[start : start + n]
            lg = buf[:n]
            gemm(hc, weight, out=lg)
            mode = 0 if (need_h or need_w) else 1
            if softcap > 0.0:  # Gemma-2: softmax over cap·tanh(logit/cap); the kernel writes the gradient w.r.t. the raw logit
                check(L.ttb_softmax_ce_capped(lg.data_ptr(), y[start : start + n].data_ptr(), loss_rows[start : start + n].data_ptr(), None, n, V, lg.stride(0), int(ignore_index), mode,
                                              float(softcap), stream_ptr()), "softmax_ce_capped")
            else:
                check(L.ttb_softmax_ce(lg.data_ptr(), y[start : start + n].data_ptr(), loss_rows[start : start + n].data_ptr(), None, n, V, lg.stride(0), int(ignore_index), mode, stream_ptr()), "softmax_ce")
            if need_h:
                gemm(lg, weight, b_mn=True, out=dh[start : start + n])
            if direct:
                gemm(lg, hc, a_mn=True, b_mn=True, out=owner._grad_buffer, accumulate=bool(owner._grad_written))
                owner._grad_written = True
            elif need_w:
                gemm(lg, hc, a_mn=True, b_mn=True, out=dw, accumulate=not single)
        ctx.save_for_backward(dh, dw)
        ctx.h_shape = hidden.shape
        ctx.w_dtype = weight.dtype
        ctx.direct = direct
        n_valid = (y != ignore_index).sum()
        ctx.mark_non_differentiable(n_valid)
        return loss_rows.sum(), n_valid

    @staticmethod
    def backward(ctx, g_loss, _g_count):
        dh, dw = ctx.saved_tensors
        # The gradients were formed for d(loss_sum) = 1; an upstream factor multiplies them.
        # With direct delivery the weight gradient already sits in the flat buffer, which is
        # only valid for an upstream factor of one (the recipes back-propagate the sum itself).
        gh = (dh * g_loss.to(dh.dtype)).view(ctx.h_shape) if dh is not None else None
        gw = (dw * g_loss).to(ctx.w_dtype) if dw is not None else None
        return gh, gw, None, None, None, None


def linear_cross_entropy(hidden, weight, labels, ignore_index: int, num_chunks: int, softcap: float = 0.0):
    if hidden.shape[-1] % 8 or weight.shape[0] % 8:
        from . import _fallback, reference

        _fallback("linear_cross_entropy", f"width {hidden.shape[-1]} or vocabulary {weight.shape[0]} is not a multiple of 8", hidden)
        return reference.linear_cross_entropy(hidden, weight, labels, ignore_index, num_chunks, softcap=softcap)
    return _LinearCE.apply(hidden, weight, labels, ignore_index, num_chunks, float(softcap))


def _softmax_ce(buf, labels, loss_out, row_scale, n, V, ignore_index, mode, softcap=0.0):
    """One launch of the softmax / cross-entropy kernel over ``buf[:n]`` (see ``loss.cu``), with the logits soft-capped when asked."""
    args = (buf.data_ptr(), labels.data_ptr(), _ptr(loss_out), _ptr(row_scale), n, V, buf.stride(0), int(ignore_index), mode)
    if softcap > 0.0:
        check(lib().ttb_softmax_ce_capped(*args, float(softcap), stream_ptr()), "softmax_ce_capped")
    else:
        check(lib().ttb_softmax_ce(*args, stream_ptr()), "softmax_ce")


class _TokenLogprobs(torch.autograd.Function):
    """Per-token log p(label) through the output projection; backward recomputes each logits
    chunk and scales the in-place softmax gradient by the incoming per-token gradient."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, num_chunks, softcap=0.0):
        D = hidden.shape[-1]
        h2 = hidden.reshape(-1, D).contiguous()
        y = labels.reshape(-1).to(torch.int64).contiguous()
        T, V = h2.shape[0], weight.shape[0]
        rows = _ce_chunk_rows(T, num_chunks)
        nll = torch.empty(T, dtype=torch.float32, device=h2.device)
        buf = torch.empty(min(rows, T), V, dtype=_BF16, device=h2.device)
        for start in range(0, T, rows):
            n = min(rows, T - start)
            gemm(h2[start : start + n], weight, out=buf[:n])
            _softmax_ce(buf, y[start : start + n], nll[start : start + n], None, n, V, ignore_index, 1, softcap)
        ctx.save_for_backward(h2, weight, y)
        ctx.meta = (ignore_index, rows, hidden.shape, labels.shape)
        ctx.softcap = float(softcap)
        return (-nll).view(labels.shape)

    @staticmethod
    def backward(ctx, g):
        h2, weight, y = ctx.saved_tensors
        ignore_index, rows, h_shape, _ = ctx.meta
        T, V = h2.shape[0], weight.shape[0]
        gs = g.reshape(-1).float().contiguous()
        need_w = ctx.needs_input_grad[1]
        dh = torch.empty_like(h2)
        dw = torch.zeros(V, h2.shape[1], dtype=torch.float32, device=h2.device) if need_w else None
        buf = torch.empty(min(rows, T), V, dtype=_BF16, device=h2.device)
        for start in range(0, T, rows):
            n = min(rows, T - start)
            hc = h2[start : start + n]
            gemm(hc, weight, out=buf[:n])
            _softmax_ce(buf, y[start : start + n], None, gs[start : start + n], n, V, ignore_index, 2, ctx.softcap)
            gemm(buf[:n], weight, b_mn=True, out=dh[start : start + n])
            if need_w:
                gemm(buf[:n], hc, a_mn=True, b_mn=True, out=dw, accumulate=True)
        return dh.view(h_shape), (dw.to(weight.dtype) if need_w else None), None, None, None, None


def token_logprobs(hidden, weight, labels, ignore_index: int, num_chunks: int, softcap: float = 0.0):
    return _TokenLogprobs.apply(hidden, weight, labels, ignore_index, num_chunks, float(softcap))


# ======================================================================= optimizer
class _MetaTable:
    """Device copy of the (param, grad, exp_avg, exp_avg_sq, master) pointer table; rebuilt
    only when a pointer changes (e.g. gradients re-allocated after ``zero_grad``)."""

    def __init__(self) -> None:
        self.key: Optional[Tuple[int, ...]] = None
        self.dev: Optional[torch.Tensor] = None
        self.n = 0
        self.chunks = 0

    def update(self, items: Sequence[Tuple[torch.Tensor, torch.Tensor, Dict[str, Any]]], device: torch.device) -> None:
        chunk = lib().ttb_optim_chunk()
        rows: List[int] = []
        total = 0
        for p, g, st in items:
            master = st.get("master")
            rows += [p.data_ptr(), g.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(), master.data_ptr() if master is not None else 0, p.numel(), total]
            total += -(-p.numel() // chunk)
        key = tuple(rows)
        if key != self.key:
            host = torch.tensor(rows, dtype=torch.int64).view(-1, 7)
            self.dev = host.to(device, non_blocking=False)
            self.key = key
        self.n = len(items)
        self.chunks = total


_tables: Dict[Tuple[int, torch.dtype], _MetaTable] = {}


def _table_for(items, tag: int) -> _MetaTable:
    dtype = items[0][0].dtype
    tbl = _tables.setdefault((tag, dtype), _MetaTable())
    tbl.update(items, items[0][0].device)
    return tbl


def adamw_multi(items, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, grad_scale: Union[float, torch.Tensor] = 1.0, tag: int = 0) -> None:
    """One kernel launch per dtype group over all ``(param, grad, state)`` triples."""
    groups: Dict[torch.dtype, list] = {}
    for it in items:
        p, g, _ = it
        if p.dtype not in (_BF16, torch.float32) or g.dtype != p.dtype or not p.is_contiguous() or not g.is_contiguous():
            raise _lib.KernelError("adamw_multi needs contiguous bf16/fp32 params with same-dtype grads")
        groups.setdefault(p.dtype, []).append(it)
    scale_dev = None
    scale_host = 1.0
    if isinstance(grad_scale, torch.Tensor):
        scale_dev = grad_scale.to(torch.float32).reshape(1)
    else:
        scale_host = float(grad_scale)
    for dtype, its in groups.items():
        step = its[0][2]["step"]
        tbl = _table_for(its, tag)
        inv_bc1 = 1.0 / (1.0 - beta1**step)
        inv_sqrt_bc2 = 1.0 / math.sqrt(1.0 - beta2**step)
        check(lib().ttb_adamw(tbl.dev.data_ptr(), tbl.n, tbl.chunks, int(dtype == _BF16), lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_sqrt_bc2, _ptr(scale_dev), scale_host, stream_ptr()), "adamw")


def adamw8bit(p: torch.Tensor, g: torch.Tensor, mq: torch.Tensor, vq: torch.Tensor, mscale: torch.Tensor, vscale: torch.Tensor, step: int, lr: float, beta1: float,
              beta2: float, eps: float, weight_decay: float, grad_scale: Union[float, torch.Tensor] = 1.0) -> None:
    """AdamW update of one tensor whose moments are stored as one-byte codes with a scale per 256 elements (``optim.cu``)."""
    if p.dtype not in (_BF16, torch.float32) or g.dtype != p.dtype or not p.is_contiguous() or not g.is_contiguous():
        raise _lib.KernelError("adamw8bit needs contiguous bf16/fp32 params with same-dtype grads")
    scale_dev, scale_host = (grad_scale.to(torch.float32).reshape(1), 1.0) if isinstance(grad_scale, torch.Tensor) else (None, float(grad_scale))
    check(lib().ttb_adamw8bit(p.data_ptr(), g.data_ptr(), mq.data_ptr(), vq.data_ptr(), mscale.data_ptr(), vscale.data_ptr(), p.numel(), int(p.dtype == _BF16), lr, beta1, beta2,
                              eps, weight_decay, 1.0 / (1.0 - beta1**step), 1.0 / math.sqrt(1.0 - beta2**step), _ptr(scale_dev), scale_host, stream_ptr()), "adamw8bit")


def grad_sumsq(items, tag: int = 1) -> torch.Tensor:
    """Sum of squared gradient entries over all items (0-d fp32 tensor, no host sync)."""
    groups: Dict[torch.dtype, list] = {}
    for it in items:
        groups.setdefault(it[0].dtype, []).append(it)
    total = None
    for dtype, its in groups.items():
        tbl = _table_for(its, tag)
        partials = torch.empty(lib().ttb_optim_grid(), dtype=torch.float32, device=its[0][0].device)
        check(lib().ttb_grad_sumsq(tbl.dev.data_ptr(), tbl.n, tbl.chunks, int(dtype == _BF16), partials.data_ptr(), stream_ptr()), "grad_sumsq")
        s = partials.sum()
        total = s if total is None else total + s
    return total
