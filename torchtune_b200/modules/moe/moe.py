"""Token-choice top-k routing and the MoE layer (parity: torchtune/modules/moe/moe.py:15-150)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ... import ops


class TokenChoiceTopKRouter(nn.Module):
    """Every token picks its ``experts_per_token`` highest-scoring experts (sigmoid scores,
    computed in fp32).  Returns, for the ``tokens·k`` (token, expert) pairs sorted by expert:
    their scores, the source token index of each pair, and the pair count per expert."""

    def __init__(self, *, gate: nn.Module, dim: int, num_experts: int, experts_per_token: int):
        super().__init__()
        self.gate, self.dim, self.num_experts, self.experts_per_token = gate, dim, num_experts, experts_per_token

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        self.pair_positions = None  # [tokens·k] position of every (token, slot) pair in expert order (CUDA kernels only)
        if ops.cuda_ops_enabled(x) and x.dtype == torch.bfloat16 and self.num_experts <= 256 and self.experts_per_token <= 8:
            # two launches: sigmoid + top-k (one warp per token), then histogram + stable sort (which also returns where every pair went)
            from ...ops._cuda import moe_route, moe_route_sort

            top_scores, selected = moe_route(self.gate(x), self.experts_per_token)
            self.selected_experts_indices = selected
            num_tokens_per_expert, order, self.pair_positions = moe_route_sort(selected.reshape(-1), self.num_experts, with_inverse=True)
            self.tokens_per_expert = num_tokens_per_expert.detach()
            return top_scores.reshape(-1)[order], order // self.experts_per_token, num_tokens_per_expert
        scores = torch.sigmoid(self.gate(x).to(torch.float32)).to(x.dtype)
        top_scores, selected = torch.topk(scores, k=self.experts_per_token, dim=1)
        self.selected_experts_indices = selected
        flat = selected.reshape(-1)
        if ops.cuda_ops_enabled(flat) and self.num_experts <= 256:
            from ...ops._cuda import moe_route_sort

            num_tokens_per_expert, order = moe_route_sort(flat, self.num_experts)  # one launch: histogram + stable sort
        else:
            num_tokens_per_expert = torch.bincount(flat, minlength=self.num_experts)
            order = torch.argsort(flat, stable=True)
        self.tokens_per_expert = num_tokens_per_expert.detach()  # load statistics (see utils.expert_load_imbalance)
        return top_scores.reshape(-1)[order], order // self.experts_per_token, num_tokens_per_expert


class MoE(nn.Module):
    """``out = shared_expert(x) + scatter_add(experts(score · gather(x)))``; scores multiply the
    expert *input* (Llama-4 convention)."""

    def __init__(self, *, experts: nn.Module, router: nn.Module, shared_expert: Optional[nn.Module] = None):
        super().__init__()
        self.experts, self.router, self.shared_expert = experts, router, shared_expert

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bs, slen, dim = x.shape
        flat = x.reshape(bs * slen, dim)
        top_scores, token_indices, num_tokens_per_expert = self.router(flat)
        inv = getattr(self.router, "pair_positions", None)
        if inv is not None and dim % 8 == 0:
            # permute·score and un-permute + sum as row kernels (every output row pulls its sources: no atomics, no index_add)
            from ...ops._cuda import moe_combine, moe_gather

            k = self.router.experts_per_token
            routed_out = self.experts(moe_gather(flat, token_indices, top_scores, inv, k), num_tokens_per_expert)
            shared = self.shared_expert(flat) if self.shared_expert is not None else None
            return moe_combine(routed_out, inv, token_indices, shared, k).reshape(bs, slen, dim)
        routed_in = flat.index_select(0, token_indices) * top_scores.reshape(-1, 1)
        routed_out = self.experts(routed_in, num_tokens_per_expert)
        out = self.shared_expert(flat) if self.shared_expert is not None else torch.zeros_like(flat)
        out = out.index_add(0, token_indices, routed_out.to(out.dtype))
        return out.reshape(bs, slen, dim)
