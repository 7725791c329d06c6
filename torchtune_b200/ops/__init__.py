"""Operator layer.

Every operator has two statements: the sm_100a CUDA kernel (``_cuda``,
compiled from ``csrc/``) used for CUDA tensors, and the plain PyTorch one in
:mod:`.reference` used on CPU and as the numerical oracle.  On a CUDA device a
missing extension is an error.  A bf16 CUDA call whose *shape or options* the
kernels do not cover takes the PyTorch statement instead; every such call is
counted in :data:`fallback_counts`, logged once per (operator, reason), and raises
:class:`KernelFallbackError` when ``TTB_STRICT=1`` (set by the benchmark and the
GPU tests) so a configuration cannot run on library or eager math unnoticed.
"""
from __future__ import annotations

import os
import warnings
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import reference
from .mask import AttentionMask

__all__ = [
    "grouped_matmul",
    "lora_linear",
    "lora_linear_nf4",
    "fp8_linear",
    "mxfp8_linear",
    "matmul",
    "linear",
    "linear_residual",
    "rms_norm",
    "rope",
    "swiglu",
    "attention",
    "linear_cross_entropy",
    "token_logprobs",
    "embedding",
    "embed_tokens",
    "AttentionMask",
    "reference",
    "cuda_ops_enabled",
]

_FORCE_REFERENCE = False

fallback_counts: Dict[Tuple[str, str], int] = {}


class KernelFallbackError(RuntimeError):
    """A bf16 CUDA operator call would have left the sm_100a kernels while ``TTB_STRICT=1``."""


def _fallback(op: str, reason: str, t: torch.Tensor) -> None:
    """Record that ``op`` runs its PyTorch statement for bf16 CUDA input ``t`` (no-op for CPU / fp32 tensors and inside
    :class:`use_reference_ops`, where the PyTorch statement is the intended one)."""
    if not (t.is_cuda and t.dtype == torch.bfloat16) or _FORCE_REFERENCE:
        return
    key = (op, reason)
    n = fallback_counts.get(key, 0)
    fallback_counts[key] = n + 1
    if os.environ.get("TTB_STRICT", "0") == "1":
        raise KernelFallbackError(f"ops.{op}: {reason} — not covered by the sm_100a kernels (TTB_STRICT=1 forbids the PyTorch fallback)")
    if n == 0:
        warnings.warn(f"ops.{op}: {reason}; running the PyTorch statement instead of the sm_100a kernel", RuntimeWarning, stacklevel=3)


class use_reference_ops:
    """Context manager that forces the PyTorch statements (used by parity tests)."""

    def __enter__(self):
        global _FORCE_REFERENCE
        self._prev = _FORCE_REFERENCE
        _FORCE_REFERENCE = True

    def __exit__(self, *exc):
        global _FORCE_REFERENCE
        _FORCE_REFERENCE = self._prev


def cuda_ops_enabled(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REFERENCE


def _native(t: torch.Tensor, dtypes=(torch.bfloat16,)) -> bool:
    return t.is_cuda and not _FORCE_REFERENCE and t.dtype in dtypes


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``; bf16 CUDA inputs run the tcgen05 GEMM (fwd, dgrad, wgrad)."""
    if _native(x) and weight.dtype == torch.bfloat16:
        from . import _cuda

        if x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
            return _cuda.linear(x, weight, bias)
        if x.shape[-1] % 8 == 0:
            # an output width that is not a multiple of 8 (a router over 4 experts, a scalar reward head): rows of zeros are
            # appended to the weight so the output row pitch is a multiple of 16 bytes, and the extra columns are cut off again;
            # autograd carries the padding and the slice through the backward pass
            n = weight.shape[0]
            pad = (-n) % 8
            y = _cuda.linear(x, F.pad(weight, (0, 0, 0, pad)), None if bias is None else F.pad(bias, (0, pad)))
            return y[..., :n]
        _fallback("linear", f"K={x.shape[-1]} is not a multiple of 8 (TMA row pitch)", x)
    return F.linear(x, weight, bias)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], residual: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T (+ bias) + residual``; bf16 CUDA inputs add the residual in the GEMM epilogue (no separate element-wise pass)."""
    if (_native(x) and weight.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16 and residual.is_cuda and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0
            and residual.shape == (*x.shape[:-1], weight.shape[0]) and os.environ.get("TTB_FUSE_RESIDUAL", "1") != "0"):
        from . import _cuda

        return _cuda.linear_residual(x, weight, bias, residual)
    return linear(x, weight, bias) + residual


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, rowwise: bool = False) -> Optional[torch.Tensor]:
    """fp8 tensor-core linear (dynamic scaling); returns ``None`` when the inputs do not qualify (not bf16 CUDA, or a dimension that
    is not a multiple of 16) so the caller can fall back to its emulation."""
    if not (_native(x) and weight.dtype == torch.bfloat16 and weight.is_contiguous()):
        return None
    tokens = x.numel() // x.shape[-1]
    if x.shape[-1] % 16 or weight.shape[0] % 16 or tokens % 16 or tokens == 0:
        return None
    from . import _cuda

    return _cuda.fp8_linear(x, weight, bias, rowwise)


def mxfp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Block-scaled (MX: e4m3 values, one power-of-two scale per 32 values along each contraction) fp8 tensor-core linear; ``None``
    when the inputs do not qualify (not bf16 CUDA, or tokens / in / out features not multiples of 32)."""
    if not (_native(x) and weight.dtype == torch.bfloat16 and weight.is_contiguous()):
        return None
    tokens = x.numel() // x.shape[-1]
    if x.shape[-1] % 32 or weight.shape[0] % 32 or tokens % 32 or tokens == 0:
        return None
    from . import _cuda

    return _cuda.mxfp8_linear(x, weight, bias)


def lora_linear(x: torch.Tensor, xd: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], lora_a: torch.Tensor, lora_b: torch.Tensor, scale: float) -> torch.Tensor:
    """``x @ weight.T (+ bias) + scale · (xd @ lora_a.T) @ lora_b.T`` — ``xd`` is the adapter branch's input (``x`` after dropout)."""
    rank = lora_a.shape[0]
    if _native(x) and weight.dtype == lora_a.dtype == lora_b.dtype == torch.bfloat16 and rank % 8 == 0 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        from . import _cuda

        return _cuda.lora_linear(x, xd, weight, bias, lora_a, lora_b, scale)
    _fallback("lora_linear", f"rank {rank} / K / N not multiples of 8 or mixed dtypes", x)
    return F.linear(x, weight, bias) + scale * F.linear(F.linear(xd, lora_a), lora_b)


def lora_linear_nf4(x: torch.Tensor, xd: torch.Tensor, nf4, bias: Optional[torch.Tensor], lora_a: torch.Tensor, lora_b: torch.Tensor, scale: float) -> Optional[torch.Tensor]:
    """:func:`lora_linear` over an NF4 base weight (``nf4``: an object with ``dequantize(dtype)``); ``None`` when the inputs do not
    qualify for the fused CUDA path."""
    rank = lora_a.shape[0]
    if _native(x) and lora_a.dtype == lora_b.dtype == torch.bfloat16 and rank % 8 == 0 and x.shape[-1] % 8 == 0 and lora_b.shape[0] % 8 == 0:
        from . import _cuda

        return _cuda.lora_linear_nf4(x, xd, nf4, bias, lora_a, lora_b, scale)
    return None


def grouped_matmul(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Expert-grouped product: rows of ``x`` ``[rows, K]`` are sorted by expert, ``counts[e]`` rows belong to expert ``e`` and are
    multiplied by ``w[e]`` (``w``: ``[E, K, N]``)."""
    if _native(x) and w.dtype == torch.bfloat16 and x.shape[0] > 0 and x.is_contiguous() and w.is_contiguous() and x.shape[1] % 8 == 0 and w.shape[2] % 8 == 0 and counts.is_cuda:
        from . import _cuda

        return _cuda.grouped_matmul(x, w, counts)
    if x.shape[0] > 0:
        _fallback("grouped_matmul", "non-contiguous operands, host-side counts or K / N not multiples of 8", x)
    outs, start = [], 0
    for e, n in enumerate(counts.tolist()):
        if n:
            outs.append(x[start : start + n] @ w[e])
        start += n
    return torch.cat(outs) if outs else x.new_zeros(0, w.shape[2])


def matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x[T, K] @ w[K, N]`` (2-D operands, ``w`` row-major as stored in grouped expert weights)."""
    if _native(x) and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.shape[0] > 0 and x.is_contiguous() and w.is_contiguous() and x.shape[1] % 8 == 0 and w.shape[1] % 8 == 0:
        from . import _cuda

        return _cuda.matmul_kn(x, w)
    if x.numel() > 0:
        _fallback("matmul", "operands are not contiguous 2-D matrices with K / N multiples of 8", x)
    return x @ w


def rms_norm(x: torch.Tensor, scale: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    if _native(x, (torch.bfloat16, torch.float32)):
        from . import _cuda

        return _cuda.rms_norm(x, scale, eps)
    return reference.rms_norm(x, scale, eps)


def rope(
    x: torch.Tensor, cache: torch.Tensor, input_pos: Optional[torch.Tensor] = None, interleaved: bool = True
) -> torch.Tensor:
    """Rotary embedding on ``[b, s, h, d]``; ``cache`` ``[max_seq, d/2, 2]`` (cos, sin) fp32."""
    if _native(x):
        from . import _cuda

        return _cuda.rope(x, cache, input_pos, interleaved)
    fn = reference.rope_interleaved if interleaved else reference.rope_half
    return fn(x, cache, input_pos)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if _native(gate):
        from . import _cuda

        return _cuda.swiglu(gate, up)
    return reference.swiglu(gate, up)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: Optional[AttentionMask] = None,
    *,
    scale: Optional[float] = None,
    softcap: float = 0.0,
    dropout_p: float = 0.0,
) -> torch.Tensor:
    """Grouped-query attention on ``[b, s, h, d]`` without materialising expanded KV heads."""
    mask = mask if mask is not None else AttentionMask(causal=False)
    if _native(q):
        from . import _cuda_attention

        why = None
        if dropout_p != 0.0:
            why = "attention dropout"
        elif q.shape[-1] not in (64, 128):
            why = f"head_dim {q.shape[-1]}"
        else:
            why = _cuda_attention.unsupported_reason(q, k, mask)
        if why is None:
            return _cuda_attention.attention(q, k, v, mask, scale, softcap)
        _fallback("attention", why, q)
    return reference.attention(
        q,
        k,
        v,
        causal=mask.causal,
        doc_ids=mask.doc_ids,
        chunk=mask.chunk,
        window=mask.window,
        bool_mask=mask.bool_mask,
        scale=scale,
        softcap=softcap,
        dropout_p=dropout_p,
    )


def linear_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    ignore_index: int = -100,
    num_chunks: int = 8,
    softcap: float = 0.0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(sum of CE, number of valid tokens)`` of ``hidden @ weight.T`` vs ``labels``; with ``softcap > 0`` the softmax runs over
    ``softcap · tanh(logits / softcap)`` (Gemma-2)."""
    if _native(hidden) and weight.dtype == torch.bfloat16:
        from . import _cuda

        return _cuda.linear_cross_entropy(hidden, weight, labels, ignore_index, num_chunks, softcap)
    return reference.linear_cross_entropy(hidden, weight, labels, ignore_index, num_chunks, softcap=softcap)


def token_logprobs(
    hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, num_chunks: int = 8, softcap: float = 0.0
) -> torch.Tensor:
    """Per-token ``log_softmax(hidden @ weight.T)[label]``; with ``softcap > 0`` over ``softcap · tanh(logits / softcap)``."""
    if _native(hidden) and weight.dtype == torch.bfloat16:
        from . import _cuda

        return _cuda.token_logprobs(hidden, weight, labels, ignore_index, num_chunks, softcap)
    return reference.token_logprobs(hidden, weight, labels, ignore_index, num_chunks, softcap=softcap)


def logit_softcap_of(model) -> float:
    """The soft cap a decoder applies to its logits (0 = none); callers that take hidden states and do the output projection
    themselves pass it on to :func:`linear_cross_entropy` / :func:`token_logprobs`."""
    core = getattr(model, "decoder", model)
    return float(getattr(core, "logit_softcap", 0.0) or 0.0)


def logits_logprobs(logits: torch.Tensor, tokens: torch.Tensor, temperature: float = 1.0) -> Optional[torch.Tensor]:
    """``log_softmax(logits / T)`` gathered at ``tokens`` (fp32, shape of ``tokens``) for bf16 CUDA logits whose vocabulary width is a
    multiple of 8, without an fp32 ``[..., V]`` intermediate; ``None`` otherwise."""
    if not (_native(logits) and logits.shape[-1] % 8 == 0 and tokens.is_cuda and tokens.dtype == torch.int64 and logits.shape[:-1] == tokens.shape and logits.numel() > 0):
        return None
    from . import _cuda

    return _cuda.logits_logprobs(logits, tokens, temperature)


def sample_tokens(logits: torch.Tensor, q: torch.Tensor, temperature: float, top_k: Optional[int]) -> Optional[torch.Tensor]:
    """Fused temperature / top-k / exponential-race draw for CUDA logits (``[..., V]`` bf16 or fp32, ``q`` fp32 of the same shape);
    int32 tokens ``[..., 1]``, or ``None`` when the inputs do not qualify."""
    if not (logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and q.is_cuda and q.dtype == torch.float32 and q.shape == logits.shape
            and logits.dim() >= 1 and logits.numel() > 0 and not _FORCE_REFERENCE):
        return None
    from . import _cuda

    V = logits.shape[-1]
    l2, q2 = logits.reshape(-1, V), q.reshape(-1, V)
    if l2.stride(1) != 1:
        l2 = l2.contiguous()
    if q2.stride(1) != 1:
        q2 = q2.contiguous()
    return _cuda.sample(l2, q2, temperature, top_k).view(*logits.shape[:-1], 1)


def kd_divergence(student_logits: torch.Tensor, teacher_logits: torch.Tensor, labels: torch.Tensor, w_fwd: float, w_rev: float,
                  ignore_index: int = -100) -> Optional[torch.Tensor]:
    """Summed distillation divergence ``w_fwd · forward-KL term + w_rev · reverse KL`` over the rows whose label is not
    ``ignore_index`` (fused kernel: both softmaxes, the loss and the student gradient in one launch); ``None`` when the inputs are
    not bf16 CUDA logits with a vocabulary width that is a multiple of 8."""
    if not (_native(student_logits) and teacher_logits.is_cuda and teacher_logits.dtype == torch.bfloat16 and student_logits.shape[-1] % 8 == 0
            and student_logits.shape == teacher_logits.shape and labels.is_cuda):
        return None
    from . import _cuda

    return _cuda.kd_divergence(student_logits, teacher_logits, labels, w_fwd, w_rev, ignore_index)


def embedding(tokens: torch.Tensor, weight: torch.Tensor, padding_idx: Optional[int] = None) -> torch.Tensor:
    """``weight[tokens]``; bf16 CUDA tables use the gather kernel and the sorted, fp32-accumulating gradient kernel."""
    if _native(weight) and tokens.is_cuda and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.is_contiguous():
        from . import _cuda

        return _cuda.embedding(tokens, weight, padding_idx)
    return F.embedding(tokens, weight, padding_idx)


def embed_tokens(module: torch.nn.Module, tokens: torch.Tensor) -> torch.Tensor:
    """Calls an embedding module; a plain ``nn.Embedding`` (no max-norm, dense gradient) is routed through :func:`embedding`."""
    if type(module) is torch.nn.Embedding and module.max_norm is None and not module.sparse and not module.scale_grad_by_freq:
        return embedding(tokens, module.weight, module.padding_idx)
    return module(tokens)
