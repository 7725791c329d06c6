"""Grouped SwiGLU experts (parity: torchtune/modules/moe/experts.py:18-290).

Weights are stored per expert as ``gate_proj``/``up_proj`` ``[E, dim, hidden]`` and ``down_proj``
``[E, hidden, dim]`` (the reference's state-dict layout).  Tokens arrive sorted by expert; expert
``e`` owns rows ``offsets[e]:offsets[e+1]``.  Every expert product runs through
:func:`torchtune_b200.ops.matmul`, i.e. the tcgen05 GEMM reading the weight in place as an
MN-major operand — no transposed copies, no padding of the token groups.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ..peft._utils import AdapterModule


def _segments(num_tokens_per_expert: torch.Tensor) -> List[int]:
    return [int(n) for n in num_tokens_per_expert.tolist()]


class GroupedExperts(nn.Module):
    def __init__(self, *, dim: int, hidden_dim: int, num_experts: int = 1, activation: Callable = F.silu):
        super().__init__()
        self.dim, self.hidden_dim, self.num_experts = dim, hidden_dim, num_experts
        self.gate_proj = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.down_proj = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.up_proj = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.act_fn = activation
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.gate_proj.is_meta:
            return
        for w in (self.gate_proj, self.down_proj, self.up_proj):
            nn.init.kaiming_uniform_(w, a=math.sqrt(5))

    def _expert(self, e: int, x: torch.Tensor) -> torch.Tensor:
        g = ops.matmul(x, self.gate_proj[e])
        u = ops.matmul(x, self.up_proj[e])
        h = ops.swiglu(g, u) if self.act_fn is F.silu else self.act_fn(g) * u
        return ops.matmul(h, self.down_proj[e])

    def forward(self, x: torch.Tensor, num_tokens_per_expert: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x``: ``[tokens·top_k, dim]`` sorted by expert (or ``[E, n, dim]`` when every expert gets
        the same number of rows and ``num_tokens_per_expert`` is ``None``)."""
        if num_tokens_per_expert is None:
            return torch.stack([self._expert(e, x[e]) for e in range(self.num_experts)])
        from .utils import should_use_grouped_mm

        if should_use_grouped_mm() and x.is_cuda and x.dtype == torch.bfloat16 and self.act_fn is F.silu and x.shape[0] > 0:
            # three grouped launches for all experts (tile → expert table built on the device: no host sync)
            g = ops.grouped_matmul(x, self.gate_proj, num_tokens_per_expert)
            u = ops.grouped_matmul(x, self.up_proj, num_tokens_per_expert)
            return ops.grouped_matmul(ops.swiglu(g, u), self.down_proj, num_tokens_per_expert)
        outs, start = [], 0
        for e, n in enumerate(_segments(num_tokens_per_expert)):
            if n:
                outs.append(self._expert(e, x[start : start + n]))
            start += n
        return torch.cat(outs) if outs else x.new_zeros(0, self.dim)


class LoRAGroupedExperts(nn.Module, AdapterModule):
    """Grouped experts with one low-rank adapter per expert and projection:
    ``W_e x + (alpha / r)·B_e A_e x`` for gate, up and down."""

    def __init__(self, *, dim: int, hidden_dim: int, rank: int, alpha: float, dropout: float = 0.0, num_experts: int = 1, activation: Callable = F.silu):
        super().__init__()
        self.dim, self.hidden_dim, self.num_experts = dim, hidden_dim, num_experts
        self.rank, self.alpha = rank, alpha
        self.gate_proj = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.down_proj = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.up_proj = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.act_fn = activation
        self.dropout = nn.Dropout(p=dropout) if dropout > 0.0 else nn.Identity()
        self.lora_gate_a = nn.Parameter(torch.empty(num_experts, dim, rank))
        self.lora_gate_b = nn.Parameter(torch.empty(num_experts, rank, hidden_dim))
        self.lora_down_a = nn.Parameter(torch.empty(num_experts, hidden_dim, rank))
        self.lora_down_b = nn.Parameter(torch.empty(num_experts, rank, dim))
        self.lora_up_a = nn.Parameter(torch.empty(num_experts, dim, rank))
        self.lora_up_b = nn.Parameter(torch.empty(num_experts, rank, hidden_dim))
        self.merged = False
        self.initialize_parameters()

    def initialize_parameters(self) -> None:
        if self.lora_gate_a.is_meta:
            return
        for a in (self.lora_gate_a, self.lora_down_a, self.lora_up_a):
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        for b in (self.lora_gate_b, self.lora_down_b, self.lora_up_b):
            nn.init.zeros_(b)

    def adapter_params(self) -> List[str]:
        return ["lora_gate_a", "lora_gate_b", "lora_down_a", "lora_down_b", "lora_up_a", "lora_up_b"]

    def _proj(self, x: torch.Tensor, w: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        base = ops.matmul(x, w)
        if getattr(self, "disabled", False):
            return base
        return base + (self.alpha / self.rank) * ((self.dropout(x) @ a) @ b)

    def _expert(self, e: int, x: torch.Tensor) -> torch.Tensor:
        g = self._proj(x, self.gate_proj[e], self.lora_gate_a[e], self.lora_gate_b[e])
        u = self._proj(x, self.up_proj[e], self.lora_up_a[e], self.lora_up_b[e])
        h = self.act_fn(g) * u
        return self._proj(h, self.down_proj[e], self.lora_down_a[e], self.lora_down_b[e])

    def forward(self, x: torch.Tensor, num_tokens_per_expert: Optional[torch.Tensor] = None) -> torch.Tensor:
        if num_tokens_per_expert is None:
            return torch.stack([self._expert(e, x[e]) for e in range(self.num_experts)])
        outs, start = [], 0
        for e, n in enumerate(_segments(num_tokens_per_expert)):
            if n:
                outs.append(self._expert(e, x[start : start + n]))
            start += n
        return torch.cat(outs) if outs else x.new_zeros(0, self.dim)
