"""Autograd wrapper of the tcgen05 flash-attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

import math
from typing import Optional

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


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lo, scale, causal):
        b, s, hq, d = q.shape
        hkv = k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty(b, hq, s, dtype=torch.float32, device=q.device)
        check(
            lib().ttb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), None if lo is None else lo.data_ptr(), b, s, hq, hkv, d, float(scale), int(causal), err_word(q.device).data_ptr(), stream_ptr()),
            "attention forward",
        )
        ctx.save_for_backward(q, k, v, o, lse, lo)
        ctx.scale, ctx.causal = scale, causal
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, lo = ctx.saved_tensors
        b, s, hq, d = q.shape
        hkv = k.shape[2]
        d_o = d_o.contiguous()
        delta = torch.empty(b, hq, s, dtype=torch.float32, device=q.device)
        dq_acc = torch.zeros(b, s, hq, d, dtype=torch.float32, device=q.device)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        check(
            lib().ttb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), None if lo is None else lo.data_ptr(), b, s, hq, hkv, d, float(ctx.scale), int(ctx.causal), err_word(q.device).data_ptr(), stream_ptr()),
            "attention backward",
        )
        return dq_acc.to(q.dtype), dk, dv, None, None, None


def attention(q, k, v, mask: AttentionMask, scale: Optional[float], softcap: float) -> torch.Tensor:
    b, s, hq, d = q.shape
    structured = mask.doc_ids is not None or mask.chunk > 0 or mask.window > 0
    if softcap > 0 or (structured and not mask.causal) or hq % k.shape[2]:
        from . import _fallback, reference

        _fallback("attention", "soft-capping" if softcap > 0 else ("structured mask without causality" if structured and not mask.causal else "query heads not a multiple of key heads"), q)
        return reference.attention(q, k, v, causal=mask.causal, doc_ids=mask.doc_ids, chunk=mask.chunk, window=mask.window, scale=scale, softcap=softcap)
    lo = lower_bounds(mask, b, s, q.device)
    return _FlashAttention.apply(q, k, v, lo, (1.0 / math.sqrt(d)) if scale is None else scale, mask.causal)
