"""Autograd wrapper of the tcgen05 flash-attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import os

import torch

from ._lib import check, err_word, lib, stream_ptr
from .mask import AttentionMask


def lower_bounds(mask: AttentionMask, b: int, s: int, device) -> Optional[torch.Tensor]:
    """Per-query first visible key index ``lo[b, s]`` (int32) for the structured mask kinds,
    or ``None`` when every key from 0 is visible.  Documents must be contiguous runs of equal
    ids (sample packing), which makes ``lo`` non-decreasing along the sequence."""
    cached = getattr(mask, "_lo_cache", None)
    if cached is not None and cached[0] == (b, s, str(device)):
        return cached[1]
    lo = None
    pos = torch.arange(s, device=device, dtype=torch.int32)
    if mask.doc_ids is not None:
        ids = mask.doc_ids.to(device)
        change = torch.ones_like(ids, dtype=torch.bool)
        change[:, 1:] = ids[:, 1:] != ids[:, :-1]
        start = torch.where(change, pos.view(1, s).expand_as(ids), torch.zeros_like(ids))
        lo = torch.cummax(start, dim=1).values.to(torch.int32)
    if mask.chunk > 0:
        c = ((pos // mask.chunk) * mask.chunk).view(1, s).expand(b, s)
        lo = c if lo is None else torch.maximum(lo, c)
    if mask.window > 0:
        w = (pos - (mask.window - 1)).clamp_min(0).view(1, s).expand(b, s)
        lo = w if lo is None else torch.maximum(lo, w)
    if lo is not None:
        lo = lo.to(torch.int32).contiguous()
    try:
        mask._lo_cache = ((b, s, str(device)), lo)
    except Exception:
        pass
    return lo


def dense_mask_bounds(m: torch.Tensor, b: int, s: int, sk: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Boolean mask (``[b, s, sk]``, ``[b, 1, s, sk]`` or anything that broadcasts to the first) → the kernel's
    ``(kmask uint8 [b, s, sk], lo, hi)`` with ``lo`` / ``hi`` the first / last visible key of every row (``sk`` / ``-1`` for
    rows that see nothing), which lets the kernel skip key blocks outside every row's range."""
    if m.dim() == 4:
        if m.shape[1] != 1:
            raise ValueError("per-head boolean attention masks are not supported")
        m = m[:, 0]
    m = m.to(torch.bool).expand(b, s, sk).contiguous()
    seen = m.any(-1)
    as_int = m.to(torch.int8)
    first = as_int.argmax(-1)
    last = sk - 1 - as_int.flip(-1).argmax(-1)
    lo = torch.where(seen, first, torch.full_like(first, sk)).to(torch.int32).contiguous()
    hi = torch.where(seen, last, torch.full_like(last, -1)).to(torch.int32).contiguous()
    return m.view(torch.uint8), lo, hi


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lo, hi, kmask, monotone, scale, causal, softcap):
        b, s, hq, d = q.shape
        sk, hkv = k.shape[1], k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty(b, hq, s, dtype=torch.float32, device=q.device)
        # head dim 128 with structured (monotone) bounds: two query tiles per CTA, probabilities kept in tensor memory
        two_tile = d == 128 and kmask is None and softcap == 0.0 and (monotone or (lo is None and hi is None)) and os.environ.get("TTB_ATTN_TWO_TILE", "1") != "0"
        if two_tile:
            check(
                lib().ttb_attn_fwd2(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _p(lo), _p(hi), b, s, sk, hq, hkv, float(scale), int(causal),
                                    err_word(q.device).data_ptr(), stream_ptr()),
                "attention forward (two query tiles)",
            )
        else:
            check(
                lib().ttb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _p(lo), _p(hi), _p(kmask), int(monotone), b, s, sk, hq, hkv, d,
                                   float(scale), int(causal), float(softcap), err_word(q.device).data_ptr(), stream_ptr()),
                "attention forward",
            )
        ctx.save_for_backward(q, k, v, o, lse, lo, hi, kmask)
        ctx.meta = (scale, causal, softcap, monotone)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, lo, hi, kmask = ctx.saved_tensors
        scale, causal, softcap, monotone = ctx.meta
        b, s, hq, d = q.shape
        sk, hkv = k.shape[1], k.shape[2]
        d_o = d_o.contiguous()
        delta = torch.empty(b, hq, s, dtype=torch.float32, device=q.device)
        dq_acc = torch.zeros(b, s, hq, d, dtype=torch.float32, device=q.device)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        check(
            lib().ttb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                               _p(lo), _p(hi), _p(kmask), int(monotone), b, s, sk, hq, hkv, d, float(scale), int(causal), float(softcap), err_word(q.device).data_ptr(), stream_ptr()),
            "attention backward",
        )
        return dq_acc.to(q.dtype), dk, dv, None, None, None, None, None, None, None


def unsupported_reason(q: torch.Tensor, k: torch.Tensor, mask: AttentionMask) -> Optional[str]:
    """Why a bf16 CUDA call cannot run on the kernels (``None`` = it can)."""
    s, sk = q.shape[1], k.shape[1]
    structured = mask.doc_ids is not None or mask.chunk > 0 or mask.window > 0
    if q.shape[2] % k.shape[2]:
        return "query heads not a multiple of key heads"
    if mask.bool_mask is None and structured and not mask.causal:
        return "structured mask without causality"
    if mask.bool_mask is None and structured and s != sk:
        return "structured mask with different query and key lengths"
    if mask.bool_mask is not None and mask.bool_mask.dim() == 4 and mask.bool_mask.shape[1] != 1:
        return "per-head boolean mask"
    return None


def attention(q, k, v, mask: AttentionMask, scale: Optional[float], softcap: float) -> torch.Tensor:
    """Self-attention with structured masks, cross-attention and cached decoding (``sk != s``), arbitrary boolean masks and
    soft-capped scores all run on the same pair of kernels; what differs is the mask description handed to them."""
    b, s, hq, d = q.shape
    sk = k.shape[1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    lo = hi = kmask = None
    monotone, causal = 1, bool(mask.causal)
    if mask.bool_mask is not None:
        cached = getattr(mask, "_dense_cache", None)
        if cached is not None and cached[0] == (b, s, sk, mask.bool_mask.data_ptr()):
            kmask, lo, hi = cached[1]
        else:
            kmask, lo, hi = dense_mask_bounds(mask.bool_mask, b, s, sk)
            try:
                mask._dense_cache = ((b, s, sk, mask.bool_mask.data_ptr()), (kmask, lo, hi))
            except Exception:
                pass
        monotone, causal = 0, False
    else:
        lo = lower_bounds(mask, b, s, q.device)
        if causal and s != sk:  # queries are the last s positions of the key sequence (bottom-right aligned causal mask)
            hi = (torch.arange(s, device=q.device, dtype=torch.int32) + (sk - s)).view(1, s).expand(b, s).contiguous()
    return _FlashAttention.apply(q, k, v, lo, hi, kmask, monotone, scale, causal, float(softcap or 0.0))
