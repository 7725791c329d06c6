"""Knowledge-distillation divergences (parity: torchtune/modules/loss/kd_losses.py:11-440).

Each loss compares student and teacher logits ``[tokens, vocab]`` token by token,
ignoring positions whose label equals ``ignore_index``; the ``*WithChunkedOutputLoss``
variants take lists of sequence chunks so only one fp32 chunk lives at a time.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F
from torch import nn


def _fused(student_logits, teacher_logits, labels, w_fwd: float, w_rev: float, ignore_index: int, normalize: bool):
    """bf16 CUDA logits: the fused divergence kernel (``None`` otherwise)."""
    from ... import ops

    total = ops.kd_divergence(student_logits, teacher_logits, labels, w_fwd, w_rev, ignore_index)
    if total is None:
        return None
    if not normalize:
        return total
    n = (labels != ignore_index).sum()
    return total / torch.clamp(n, min=1)


def _masked_token_mean(per_token: torch.Tensor, mask: torch.Tensor, normalize: bool) -> torch.Tensor:
    total = -(per_token * mask).sum()
    if not normalize:
        return total
    n = mask.sum()
    if n == 0:
        return per_token.new_zeros(())
    return total / n


class ForwardKLLoss(nn.Module):
    """``KL(teacher || student)`` up to the teacher-entropy constant: ``-Σ p_t log p_s``."""

    def __init__(self, ignore_index: int = -100):
        super().__init__()
        self.ignore_index = ignore_index

    def forward(self, student_logits, teacher_logits, labels, normalize: bool = True) -> torch.Tensor:
        fused = _fused(student_logits, teacher_logits, labels, 1.0, 0.0, self.ignore_index, normalize)
        if fused is not None:
            return fused
        t_prob = F.softmax(teacher_logits.float(), dim=-1)
        s_logp = F.log_softmax(student_logits.float(), dim=-1)
        inf_mask = torch.isinf(student_logits)
        x = torch.sum(torch.masked_fill(t_prob * s_logp, inf_mask, 0), dim=-1).view(-1)
        mask = (labels != self.ignore_index).int().view(-1)
        return _masked_token_mean(x, mask, normalize)


class ReverseKLLoss(nn.Module):
    """``KL(student || teacher)``: ``Σ p_s (log p_s - log p_t)``."""

    def __init__(self, ignore_index: int = -100):
        super().__init__()
        self.ignore_index = ignore_index

    def forward(self, student_logits, teacher_logits, labels, normalize: bool = True) -> torch.Tensor:
        fused = _fused(student_logits, teacher_logits, labels, 0.0, 1.0, self.ignore_index, normalize)
        if fused is not None:
            return fused
        s_prob = F.softmax(student_logits.float(), dim=-1)
        s_logp = F.log_softmax(student_logits.float(), dim=-1)
        t_logp = F.log_softmax(teacher_logits.float(), dim=-1)
        inf_mask = torch.isinf(student_logits) | torch.isinf(teacher_logits)
        prod = torch.masked_fill(s_prob * t_logp, inf_mask, 0) - torch.masked_fill(s_prob * s_logp, inf_mask, 0)
        x = prod.sum(-1).view(-1)
        mask = (labels != self.ignore_index).int().view(-1)
        return _masked_token_mean(x, mask, normalize)


class SymmetricKLLoss(nn.Module):
    """``sym_kd_ratio * forward KL + (1 - sym_kd_ratio) * reverse KL``."""

    def __init__(self, sym_kd_ratio: float = 0.5, ignore_index: int = -100):
        super().__init__()
        self.ignore_index = ignore_index
        self.sym_kd_ratio = sym_kd_ratio
        self.fkl = ForwardKLLoss(ignore_index)
        self.rkl = ReverseKLLoss(ignore_index)

    def forward(self, student_logits, teacher_logits, labels, normalize: bool = True) -> torch.Tensor:
        fused = _fused(student_logits, teacher_logits, labels, self.sym_kd_ratio, 1.0 - self.sym_kd_ratio, self.ignore_index, normalize)
        if fused is not None:
            return fused
        return self.sym_kd_ratio * self.fkl(student_logits, teacher_logits, labels, normalize) + (
            1 - self.sym_kd_ratio
        ) * self.rkl(student_logits, teacher_logits, labels, normalize)


class _ChunkedKD(nn.Module):
    def __init__(self, inner: nn.Module, num_output_chunks: int, ignore_index: int):
        super().__init__()
        self.num_output_chunks = num_output_chunks
        self.ignore_index = ignore_index
        self.inner = inner

    def forward(self, student_logits: List[torch.Tensor], teacher_logits: List[torch.Tensor], labels: torch.Tensor) -> torch.Tensor:
        t_flat = [c.reshape(-1, c.size(-1)) for c in teacher_logits]
        s_flat = [c.reshape(-1, c.size(-1)) for c in student_logits]
        n = (labels != self.ignore_index).sum()
        lbl = [c.reshape(-1) for c in labels.chunk(self.num_output_chunks, dim=1)]
        total = 0.0
        for s, t, l in zip(s_flat, t_flat, lbl):
            total = total + self.inner(s, t, l, normalize=False)
        return total / torch.clamp(n, min=1) if n > 0 else total * 0


class ForwardKLWithChunkedOutputLoss(_ChunkedKD):
    def __init__(self, num_output_chunks: int = 8, ignore_index: int = -100):
        super().__init__(ForwardKLLoss(ignore_index), num_output_chunks, ignore_index)


class ReverseKLWithChunkedOutputLoss(_ChunkedKD):
    def __init__(self, num_output_chunks: int = 8, ignore_index: int = -100):
        super().__init__(ReverseKLLoss(ignore_index), num_output_chunks, ignore_index)


class SymmetricKLWithChunkedOutputLoss(_ChunkedKD):
    def __init__(self, num_output_chunks: int = 8, sym_kd_ratio: float = 0.5, ignore_index: int = -100):
        super().__init__(SymmetricKLLoss(sym_kd_ratio, ignore_index), num_output_chunks, ignore_index)
        self.sym_kd_ratio = sym_kd_ratio
