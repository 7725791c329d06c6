"""Plain PyTorch statements of every operator in :mod:`torchtune_b200.ops`.

These run on any device, compute in fp32 where the CUDA kernels do, and are
(a) the CPU execution path and (b) the numerical oracle for the sm_100a
kernels.  Each function cites the reference framework code whose math it
restates.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, scale: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """fp32 ``x * rsqrt(mean(x^2) + eps)`` cast back, then ``* scale``
    (torchtune/modules/rms_norm.py:28-60)."""
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)
    return y if scale is None else y * scale


def rope_interleaved(x: torch.Tensor, cache: torch.Tensor, input_pos: Optional[torch.Tensor]) -> torch.Tensor:
    """Rotate pairs ``(x[2i], x[2i+1])``; ``x`` is ``[b, s, h, d]``, ``cache`` is
    ``[max_seq, d/2, 2]`` of (cos, sin) (torchtune/modules/position_embeddings.py:69-122)."""
    b, s, h, d = x.shape
    rc = cache[:s] if input_pos is None else cache[input_pos]
    rc = rc.view(-1, s, 1, d // 2, 2)
    xs = x.float().reshape(b, s, h, d // 2, 2)
    out = torch.stack(
        [xs[..., 0] * rc[..., 0] - xs[..., 1] * rc[..., 1], xs[..., 1] * rc[..., 0] + xs[..., 0] * rc[..., 1]], -1
    )
    return out.flatten(3).type_as(x)


def rope_half(x: torch.Tensor, cache: torch.Tensor, input_pos: Optional[torch.Tensor]) -> torch.Tensor:
    """Half-split ("HF") rotation: pairs ``(x[i], x[i + d/2])``
    (torchtune/models/qwen2/_positional_embeddings.py:14-119).  ``cache`` is
    ``[max_seq, d/2, 2]`` of (cos, sin)."""
    b, s, h, d = x.shape
    rc = cache[:s] if input_pos is None else cache[input_pos]
    rc = rc.view(-1, s, 1, d // 2, 2)
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2 :]
    cos, sin = rc[..., 0], rc[..., 1]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).type_as(x)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (torchtune/modules/feed_forward.py:50-53)."""
    return F.silu(gate) * up


def dense_mask(
    b: int,
    sq: int,
    skv: int,
    device: torch.device,
    causal: bool,
    doc_ids: Optional[torch.Tensor] = None,
    chunk: int = 0,
    window: int = 0,
    q_offset: int = 0,
) -> Optional[torch.Tensor]:
    """Boolean ``[b, 1, sq, skv]`` mask (True = attend) for the structured mask kinds."""
    if not causal and doc_ids is None and chunk <= 0 and window <= 0:
        return None
    qi = torch.arange(sq, device=device).view(1, sq, 1) + q_offset
    ki = torch.arange(skv, device=device).view(1, 1, skv)
    m = torch.ones(1, sq, skv, dtype=torch.bool, device=device)
    if causal:
        m = m & (ki <= qi)
    if chunk > 0:
        m = m & ((qi // chunk) == (ki // chunk))
    if window > 0:
        m = m & ((qi - ki) < window)
    if doc_ids is not None:
        m = m & (doc_ids.view(b, sq, 1) == doc_ids.view(b, 1, skv))
    return m.expand(b, sq, skv).unsqueeze(1)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = True,
    doc_ids: Optional[torch.Tensor] = None,
    chunk: int = 0,
    window: int = 0,
    bool_mask: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    softcap: float = 0.0,
    dropout_p: float = 0.0,
) -> torch.Tensor:
    """``softmax(q k^T * scale + mask) v`` on ``[b, s, h, d]`` tensors with grouped
    KV heads: query head ``h`` reads KV head ``h // (hq / hkv)``
    (torchtune/modules/attention.py:284-299; masks attention_utils.py:133-182,
    models/llama4/_chunked_attention.py:39-49).  Rows with no allowed key give 0."""
    b, sq, hq, d = q.shape
    skv, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3).reshape(b, hkv, g, sq, d)
    kf = k.float().permute(0, 2, 1, 3).unsqueeze(2)
    vf = v.float().permute(0, 2, 1, 3).unsqueeze(2)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap > 0:
        s = torch.tanh(s / softcap) * softcap
    if bool_mask is not None:
        m = bool_mask if bool_mask.dim() == 4 else bool_mask.unsqueeze(1)
    else:
        m = dense_mask(b, sq, skv, q.device, causal, doc_ids, chunk, window, q_offset=skv - sq if causal else 0)
    if m is not None:
        s = s.masked_fill(~m.unsqueeze(2), float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0:
        p = F.dropout(p, dropout_p)
    o = torch.matmul(p, vf)
    return o.reshape(b, hq, sq, d).permute(0, 2, 1, 3).to(q.dtype).contiguous()


def linear_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    ignore_index: int = -100,
    num_chunks: int = 8,
    bias: Optional[torch.Tensor] = None,
    softcap: float = 0.0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum of token cross entropies of ``hidden @ weight.T`` (soft-capped at ``softcap`` when that is positive) without keeping the
    ``[T, V]`` logits: tokens are processed in ``num_chunks`` pieces, logits upcast
    to fp32 (torchtune/modules/loss/cross_entropy_loss.py:87-188).
    Returns ``(loss_sum fp32, n_valid int64)``."""
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    total = h.new_zeros((), dtype=torch.float32)
    for hc, yc in zip(h.tensor_split(num_chunks), y.tensor_split(num_chunks)):
        if hc.shape[0] == 0:
            continue
        logits = F.linear(hc, weight, bias).float()
        if softcap > 0.0:
            logits = torch.tanh(logits / softcap) * softcap
        total = total + F.cross_entropy(logits, yc, reduction="sum", ignore_index=ignore_index)
    return total, (y != ignore_index).sum()


def token_logprobs(
    hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, num_chunks: int = 8, softcap: float = 0.0
) -> torch.Tensor:
    """Per-token ``log_softmax(hidden @ weight.T)[label]`` (0 where ignored) without the
    full logits tensor; the building block of the DPO sequence log-prob
    (torchtune/rlhf/sequence_processing.py:138-178)."""
    shape = labels.shape
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    outs = []
    for hc, yc in zip(h.tensor_split(num_chunks), y.tensor_split(num_chunks)):
        if hc.shape[0] == 0:
            continue
        logits = F.linear(hc, weight).float()
        if softcap > 0.0:
            logits = torch.tanh(logits / softcap) * softcap
        valid = yc != ignore_index
        lp = torch.log_softmax(logits, -1).gather(-1, yc.clamp_min(0).unsqueeze(-1)).squeeze(-1)
        outs.append(torch.where(valid, lp, torch.zeros_like(lp)))
    return torch.cat(outs).view(shape)


ADAMW8BIT_BLOCK = 256


def adamw8bit_decode(mq: torch.Tensor, vq: torch.Tensor, mscale: torch.Tensor, vscale: torch.Tensor, numel: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 moments from their one-byte codes: ``m = sign(q)·(|q|/127)²·scale`` and ``v = (q/255)⁴·scale`` with one scale per block
    of 256 elements (the block's largest magnitude)."""
    idx = torch.arange(numel, device=mq.device) // ADAMW8BIT_BLOCK
    um = mq.float().abs() / 127.0
    m = torch.sign(mq.float()) * um * um * mscale[idx]
    uv = vq.float() / 255.0
    v = (uv * uv) * (uv * uv) * vscale[idx]
    return m, v


def adamw8bit_step(p: torch.Tensor, g: torch.Tensor, mq: torch.Tensor, vq: torch.Tensor, mscale: torch.Tensor, vscale: torch.Tensor, step: int, lr: float,
                   beta1: float, beta2: float, eps: float, weight_decay: float, grad_scale: float = 1.0) -> None:
    """AdamW with 8-bit moments (flat views of all tensors; statement of ``optim.cu::adamw8bit_kernel``)."""
    n = p.numel()
    pf, gf = p.reshape(-1).float(), g.reshape(-1).float() * grad_scale
    m, v = adamw8bit_decode(mq, vq, mscale, vscale, n)
    m = beta1 * m + (1 - beta1) * gf
    v = beta2 * v + (1 - beta2) * gf * gf
    bc1, bc2 = 1 - beta1**step, 1 - beta2**step
    pf = pf * (1 - lr * weight_decay) - (lr / bc1) * m / (v.sqrt() / math.sqrt(bc2) + eps)
    nb = mscale.numel()
    pad = nb * ADAMW8BIT_BLOCK - n
    m_max = torch.nn.functional.pad(m.abs(), (0, pad)).view(nb, -1).amax(1)
    v_max = torch.nn.functional.pad(v, (0, pad)).view(nb, -1).amax(1)
    idx = torch.arange(n, device=p.device) // ADAMW8BIT_BLOCK
    inv_m = torch.where(m_max > 0, 1.0 / m_max, torch.zeros_like(m_max))[idx]
    inv_v = torch.where(v_max > 0, 1.0 / v_max, torch.zeros_like(v_max))[idx]
    mq.copy_((torch.sign(m) * torch.round(127.0 * (m.abs() * inv_m).sqrt())).to(torch.int8))
    vq.copy_(torch.round(255.0 * (v * inv_v).sqrt().sqrt()).to(torch.uint8))
    mscale.copy_(m_max)
    vscale.copy_(v_max)
    p.copy_(pf.view_as(p))


def adamw_step(
    p: torch.Tensor,
    g: torch.Tensor,
    m: torch.Tensor,
    v: torch.Tensor,
    step: int,
    lr: float,
    beta1: float,
    beta2: float,
    eps: float,
    weight_decay: float,
    grad_scale: float = 1.0,
    master: Optional[torch.Tensor] = None,
) -> None:
    """Decoupled-weight-decay Adam, fp32 math, state kept in the tensors' own dtype
    (``torch.optim.AdamW`` semantics)."""
    gf = g.float() * grad_scale
    pf = (master if master is not None else p).float()
    mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
    vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    pf = pf * (1 - lr * weight_decay)
    denom = (vf.sqrt() / math.sqrt(bc2)).add_(eps)
    pf = pf - (lr / bc1) * (mf / denom)
    m.copy_(mf)
    v.copy_(vf)
    if master is not None:
        master.copy_(pf)
    p.copy_(pf)


# ---------------------------------------------------------------------------
# NF4 (4-bit NormalFloat, arXiv 2305.14314) with double-quantised scales
# ---------------------------------------------------------------------------
NF4_CODEBOOK = (
    -1.0,
    -0.6961928009986877,
    -0.5250730514526367,
    -0.39491748809814453,
    -0.28444138169288635,
    -0.18477343022823334,
    -0.09105003625154495,
    0.0,
    0.07958029955625534,
    0.16093020141124725,
    0.24611230194568634,
    0.33791524171829224,
    0.44070982933044434,
    0.5626170039176941,
    0.7229568362236023,
    1.0,
)


def nf4_quantize(weight: torch.Tensor, block_size: int = 64, scaler_block_size: int = 256):
    """Quantise to NF4: per-``block_size`` absmax scales; the scales themselves are
    mean-centred and stored as int8 per ``scaler_block_size`` group with one fp32
    factor per group.  Returns ``(packed uint8 [numel/2], scaler_q int8 [n_blocks],
    scaler_factor fp32 [n_groups], scaler_mean fp32 scalar)``."""
    n = weight.numel()
    assert n % block_size == 0, "numel must be a multiple of the NF4 block size"
    n_blocks = n // block_size
    assert n_blocks % scaler_block_size == 0, "block count must be a multiple of the scaler block size"
    w = weight.detach().float().reshape(n_blocks, block_size)
    absmax = w.abs().amax(dim=1)
    mean = absmax.mean()
    centred = (absmax - mean).view(-1, scaler_block_size)
    gmax = centred.abs().amax(dim=1, keepdim=True)
    factor = 127.0 / gmax.clamp_min(1e-30)
    sq = torch.round(centred * factor).clamp(-128, 127).to(torch.int8)
    # quantise against the *dequantised* scales so the round trip is self-consistent
    scales = (sq.float() / factor).view(-1) + mean
    code = torch.tensor(NF4_CODEBOOK, dtype=torch.float32, device=weight.device)
    wn = (w / scales.clamp_min(1e-30).unsqueeze(1)).clamp(-1, 1)
    idx = (wn.unsqueeze(-1) - code).abs().argmin(-1).to(torch.uint8).view(-1)
    packed = (idx[0::2] << 4) | idx[1::2]
    return packed, sq.view(-1), factor.view(-1).float(), mean.float()


def nf4_dequantize(
    packed: torch.Tensor,
    scaler_q: torch.Tensor,
    scaler_factor: torch.Tensor,
    scaler_mean: torch.Tensor,
    shape,
    block_size: int = 64,
    scaler_block_size: int = 256,
    dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    code = torch.tensor(NF4_CODEBOOK, dtype=torch.float32, device=packed.device)
    hi = (packed >> 4).long()
    lo = (packed & 0xF).long()
    idx = torch.stack([hi, lo], -1).view(-1)
    scales = (scaler_q.float().view(-1, scaler_block_size) / scaler_factor.view(-1, 1)).view(-1) + scaler_mean
    w = code[idx].view(-1, block_size) * scales.unsqueeze(1)
    return w.view(shape).to(dtype)


# ----------------------------------------------------------------------------- MX (block-scaled) fp8
MX_BLOCK = 32


def mx_quantize(x: torch.Tensor, transpose: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """OCP MX quantisation of a 2-D tensor to e4m3 with one power-of-two scale per 32 values of the last dimension
    (of ``x.T`` when ``transpose``).  Returns ``(q, e)``: ``q`` fp32 values on the e4m3 grid (same shape as the operand) and
    ``e`` the biased scale exponents (uint8, ``[rows, k / 32]``); the operand is ``q * 2^(e - 127)`` blockwise.
    Scale rule: ``2^(floor(log2 amax) - 8)``; quotients round to nearest even and saturate at +-448; an all-zero block gets
    exponent byte 0."""
    v = x.detach().float()
    if transpose:
        v = v.t()
    rows, k = v.shape
    if k % MX_BLOCK:
        raise ValueError(f"the blocked dimension ({k}) must be a multiple of {MX_BLOCK}")
    blocks = v.reshape(rows, k // MX_BLOCK, MX_BLOCK)
    amax = blocks.abs().amax(-1)
    _, ex = torch.frexp(amax)  # amax = m * 2^ex with m in [0.5, 1)  =>  floor(log2 amax) = ex - 1
    e = (ex - 1 - 8).clamp(-127, 127)
    scale = torch.ldexp(torch.ones_like(amax), e)
    q = (blocks / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    nz = (amax > 0).unsqueeze(-1)
    q = torch.where(nz, q, torch.zeros_like(q))
    e_byte = torch.where(amax > 0, e + 127, torch.zeros_like(e)).to(torch.uint8)
    return q.reshape(rows, k), e_byte


def mx_dequantize(q: torch.Tensor, e_byte: torch.Tensor) -> torch.Tensor:
    rows, k = q.shape
    scale = torch.ldexp(torch.ones(e_byte.shape, dtype=torch.float32, device=q.device), e_byte.to(torch.int32) - 127)
    return (q.reshape(rows, k // MX_BLOCK, MX_BLOCK) * scale.unsqueeze(-1)).reshape(rows, k)


def mx_roundtrip(x: torch.Tensor, transpose: bool = False) -> torch.Tensor:
    """Quantise and dequantise (fp32 result, shape of the operand)."""
    return mx_dequantize(*mx_quantize(x, transpose))
