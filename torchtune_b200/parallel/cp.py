"""Context parallelism: the sequence is split over the ranks everywhere except inside attention.

The reference's context parallelism (torchtune/training/_distributed.py:811-886) shards every batch tensor along the
sequence and swaps SDPA for a ring attention that rotates K/V shards (all-gather or all-to-all rotation); it cannot be
combined with block masks (:860-870).  On an NVSwitch fabric every peer is one hop away at full bandwidth, so instead of
a ring this build re-partitions *around* attention (the all-to-all head/sequence exchange): projections, norms, MLP and
the loss work on ``s / cp`` tokens; right before attention ``q, k, v`` go from ``[b, s/cp, h, d]`` to
``[b, s, h/cp, d]`` (one all-to-all each), the unchanged tcgen05 attention kernel sees whole sequences for a subset of
heads — so packed / chunked / sliding-window masks keep working — and the output goes back with one more all-to-all.
Rank ``r`` of a group owns tokens ``[r·s/cp, (r+1)·s/cp)``.

The exchanges are autograd functions (each is the other's backward).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
from torch import nn


def _all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """``x``: ``[world, ...]`` contiguous; chunk ``i`` goes to rank ``i``; returns ``[world(src), ...]``."""
    out = torch.empty_like(x)
    if x.device.type == "cpu" and x.dtype == torch.bfloat16:
        xf, of = x.float(), out.float()
        dist.all_to_all_single(of, xf, group=group)
        return of.to(torch.bfloat16)
    dist.all_to_all_single(out, x, group=group)
    return out


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp: "ContextParallelContext"):
        ctx.cp = cp
        return cp._seq_to_heads(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.cp._heads_to_seq(g.contiguous()), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp: "ContextParallelContext"):
        ctx.cp = cp
        return cp._heads_to_seq(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.cp._seq_to_heads(g.contiguous()), None


class ContextParallelContext:
    def __init__(self, group=None, *, world: Optional[int] = None, rank: Optional[int] = None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)

    # raw exchanges ---------------------------------------------------------------------
    def _seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        b, s_l, h, d = x.shape
        w = self.world
        send = x.reshape(b, s_l, w, h // w, d).permute(2, 0, 1, 3, 4).contiguous()
        recv = _all_to_all(send, self.group)  # [src rank = sequence block, b, s_l, h/w, d]
        return recv.permute(1, 0, 2, 3, 4).reshape(b, w * s_l, h // w, d)

    def _heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        b, s, h_l, d = x.shape
        w = self.world
        send = x.reshape(b, w, s // w, h_l, d).permute(1, 0, 2, 3, 4).contiguous()
        recv = _all_to_all(send, self.group)  # [src rank = head group, b, s_l, h_l, d]
        return recv.permute(1, 2, 0, 3, 4).reshape(b, s // w, w * h_l, d)

    # differentiable API ----------------------------------------------------------------
    def seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """``[b, s/cp, h, d]`` → ``[b, s, h/cp, d]``.  With fewer heads than ranks (grouped-query K/V) heads are repeated so that
        every rank receives the K/V head its query heads use."""
        if self.world == 1:
            return x
        h = x.shape[2]
        if h % self.world:
            if self.world % h:
                raise ValueError(f"context parallel size {self.world} and {h} heads: one must divide the other")
            x = x.repeat_interleave(self.world // h, dim=2)
        return _SeqToHeads.apply(x, self)

    def heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.world == 1 else _HeadsToSeq.apply(x, self)

    # batch ----------------------------------------------------------------------------
    def shard_seq(self, t: torch.Tensor, dim: int = 1) -> torch.Tensor:
        n = t.shape[dim]
        if n % self.world:
            raise ValueError(f"sequence length {n} is not divisible by the context-parallel size {self.world}")
        step = n // self.world
        return t.narrow(dim, self.rank * step, step)

    def shard_batch(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        """Slice ``tokens``, ``labels`` and ``input_pos`` to this rank's tokens; the mask keeps describing whole sequences.
        Positions are made explicit because a shard no longer starts at position 0."""
        if self.world == 1:
            return batch
        tokens = batch["tokens"]
        if batch.get("input_pos") is None:
            batch["input_pos"] = torch.arange(tokens.shape[1], device=tokens.device).unsqueeze(0).expand(tokens.shape[0], -1)
        for key in ("tokens", "labels", "input_pos"):
            if batch.get(key) is not None:
                batch[key] = self.shard_seq(batch[key]).contiguous()
        return batch


def context_parallelize(model: nn.Module, cp: ContextParallelContext) -> nn.Module:
    """Attach ``cp`` to every self-attention module of ``model`` (in place)."""
    from ..modules.attention import MultiHeadAttention

    n = 0
    for m in model.modules():
        if isinstance(m, MultiHeadAttention):
            if m.num_heads % cp.world:
                raise ValueError(f"{m.num_heads} attention heads are not divisible by the context-parallel size {cp.world}")
            m.context_parallel = cp
            n += 1
    if n == 0:
        raise ValueError("no attention modules found")
    model._cp = cp
    return model
