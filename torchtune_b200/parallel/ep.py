"""Expert parallelism: the experts of every MoE layer are spread over the ranks and routed token rows travel over
NVLink peer memory.

The reference has no expert parallelism (its MoE layer, torchtune/modules/moe/moe.py:111-186, runs all experts on the
device that holds the tokens; torchtune/modules/moe/indices.py:144-217 prepares the permutation an all-to-all based
design would need).  The design here removes the all-to-all and the second permutation:

1. every rank routes its own tokens and publishes its per-expert pair counts in a peer-visible buffer;
2. ``plan``: one kernel reads all ranks' counts and computes, for each local (token, expert) pair, the rank that owns the
   expert and the *final expert-major row* of that pair in the owner's input buffer;
3. ``push`` (dispatch): one kernel gathers the token row, multiplies by the router score and stores it straight into that
   row on the owner (plain peer stores) — permute + all-to-all + re-permute in one pass;
4. the owner runs its local experts as grouped tcgen05 GEMMs over the received rows (ragged, device-resident counts);
5. ``pull`` (combine): one kernel loads every pair's result row from the owner (plain peer loads); the rows are then
   summed per token.

The backward pass is the mirror image (gradient rows are pushed where the forward pulled, and pulled where it pushed).
Ordering between ranks uses stream-ordered barriers (a 4-byte all-reduce); nothing waits inside a kernel and the host
never synchronises.  Without CUDA the same interface runs on gloo collectives so the logic is testable on CPU.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional

import os

import torch
import torch.distributed as dist
from torch import nn

from .fabric import PeerBuffer

_BF16 = torch.bfloat16


def _declare(L) -> None:
    if getattr(L, "_ep_declared", False):
        return
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    pvp = ctypes.POINTER(vp)
    L.ttb_ep_plan.argtypes = [pvp, i32, i32, i32, i64, vp, vp, vp, vp, vp]
    L.ttb_ep_push.argtypes = [vp, vp, vp, vp, vp, pvp, i32, i64, i32, i64, vp]
    L.ttb_ep_pull.argtypes = [pvp, i32, vp, vp, vp, i64, i32, i64, vp]
    for fn in (L.ttb_ep_plan, L.ttb_ep_push, L.ttb_ep_pull):
        fn.restype = i32
    L._ep_declared = True


@dataclass
class EpPlan:
    dest_rank: torch.Tensor  # int32 [pairs]
    dest_row: torch.Tensor  # int32 [pairs]
    recv_counts: torch.Tensor  # int64 [experts_per_rank] rows this rank receives per local expert
    n_pairs: int


class ExpertParallelContext:
    """Peer buffers and exchange kernels for one expert-parallel group.

    ``max_pairs`` is the largest number of routed (token, expert) pairs a rank produces per MoE call
    (tokens · experts_per_token).  ``capacity_factor`` bounds the rows a rank can receive to
    ``capacity_factor · max_pairs``; ``None`` sizes the buffers for the worst case (every pair of every rank lands on
    one rank), so no pair is ever dropped.  Pairs beyond a bounded capacity are dropped (their result is zero)."""

    def __init__(self, device: torch.device, group=None, *, num_experts: int, dim: int, max_pairs: int, capacity_factor: Optional[float] = None):
        self.device, self.group = device, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by the expert-parallel size ({self.world})")
        self.num_experts, self.dim, self.max_pairs = num_experts, dim, int(max_pairs)
        self.experts_per_rank = num_experts // self.world
        cap = self.world * self.max_pairs if capacity_factor is None else int(capacity_factor * self.max_pairs)
        self.capacity = max(128, min(cap, self.world * self.max_pairs))
        self.cuda = device.type == "cuda"
        self._token = torch.zeros(1, device=device)
        if self.cuda:
            from ..ops._lib import lib

            _declare(lib())
            self._counts = PeerBuffer(num_experts * 8, device, group)
            self._recv = PeerBuffer(self.capacity * dim * 2, device, group)
            self._result = PeerBuffer(self.capacity * dim * 2, device, group)
            # barriers between the ranks are a flag exchange over peer memory: store the next epoch into every peer's flag array
            # (release), then wait — bounded — until every peer's entry has arrived (acquire); in stream order, no collective library
            from .dp import _declare_dp

            _declare_dp(lib())
            self._flags = PeerBuffer(self.world * lib().ttb_dp_max_buckets() * 4, device, group) if self.world > 1 else None
            self._epoch = 0
        else:
            self._recv_cpu = torch.zeros(self.capacity, dim)
            self._result_cpu = torch.zeros(self.capacity, dim)

    # ------------------------------------------------------------------ plumbing
    def barrier(self) -> None:
        if self.world == 1:
            return
        if self.cuda and self._flags is not None and os.environ.get("TTB_EP_FLAG_BARRIER", "1") != "0":
            from ..ops._lib import check, err_word, lib, stream_ptr

            L = lib()
            self._epoch += 1
            check(L.ttb_dp_signal(self._flags.pointer_array(), self.world, self.rank, 0, self._epoch, stream_ptr()), "ep barrier (signal)")
            check(L.ttb_dp_wait(self._flags.local_ptr, self.world, self.rank, 0, self._epoch, err_word(self.device).data_ptr(), stream_ptr()), "ep barrier (wait)")
            return
        dist.all_reduce(self._token, group=self.group)

    def close(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            self.barrier()
            torch.cuda.synchronize(self.device)  # the flag barrier is enqueued work: it must have run before the buffers go away
            for b in (self._counts, self._recv, self._result, self._flags):
                if b is not None:
                    b.close()

    def recv_rows(self, dtype: torch.dtype) -> torch.Tensor:
        """Private copy of the rows other ranks pushed here (``[capacity, dim]``; rows past the received count are unspecified)."""
        if self.cuda:
            return self._recv.tensor(_BF16, self.capacity * self.dim).view(self.capacity, self.dim).clone()
        return self._recv_cpu.to(dtype).clone()

    def publish_result(self, rows: torch.Tensor) -> None:
        """Make ``rows`` (``[capacity, dim]``, expert-major) visible to the ranks that will pull them."""
        n = min(rows.shape[0], self.capacity)  # the loop form of the experts returns only the received rows
        if self.cuda:
            self._result.tensor(_BF16, self.capacity * self.dim).view(self.capacity, self.dim)[:n].copy_(rows[:n])
        else:
            self._result_cpu = torch.zeros(self.capacity, self.dim)
            self._result_cpu[:n] = rows[:n].detach().float()
        self.barrier()

    # ------------------------------------------------------------------ plan
    def plan(self, counts: torch.Tensor, n_pairs: int) -> EpPlan:
        """``counts``: int64 ``[num_experts]`` pairs of this rank per (global) expert, pairs sorted by expert."""
        if n_pairs > self.max_pairs:
            raise ValueError(f"{n_pairs} routed pairs exceed the context's max_pairs ({self.max_pairs})")
        if not self.cuda:
            return self._plan_cpu(counts, n_pairs)
        from ..ops._lib import check, lib, stream_ptr

        self._counts.tensor(torch.int64, self.num_experts).copy_(counts)
        self.barrier()  # every rank's counts are in place
        dest_rank = torch.empty(n_pairs, dtype=torch.int32, device=self.device)
        dest_row = torch.empty(n_pairs, dtype=torch.int32, device=self.device)
        recv_counts = torch.empty(self.experts_per_rank, dtype=torch.int64, device=self.device)
        recv_total = torch.empty(1, dtype=torch.int32, device=self.device)
        check(lib().ttb_ep_plan(self._counts.pointer_array(), self.world, self.rank, self.num_experts, n_pairs, dest_rank.data_ptr(), dest_row.data_ptr(),
                                recv_counts.data_ptr(), recv_total.data_ptr(), stream_ptr()), "ep_plan")
        if self.capacity < self.world * self.max_pairs:  # bounded capacity: experts only see the rows that fit
            recv_counts = _clip_counts(recv_counts, self.capacity)
        return EpPlan(dest_rank, dest_row, recv_counts, n_pairs)

    def _plan_cpu(self, counts: torch.Tensor, n_pairs: int) -> EpPlan:
        all_counts = [torch.empty_like(counts) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(all_counts, counts.contiguous(), group=self.group)
        else:
            all_counts = [counts]
        c = torch.stack(all_counts)  # [world, E]
        epr = self.experts_per_rank
        total = c.sum(0)
        before = c[: self.rank].sum(0)
        row0 = total.view(self.world, epr).cumsum(1) - total.view(self.world, epr)
        base = row0.reshape(-1) + before
        expert = torch.repeat_interleave(torch.arange(self.num_experts), c[self.rank])
        first = c[self.rank].cumsum(0) - c[self.rank]
        pos = torch.arange(n_pairs) - first[expert]
        recv_counts = total.view(self.world, epr)[self.rank].clone()
        if self.capacity < self.world * self.max_pairs:
            recv_counts = _clip_counts(recv_counts, self.capacity)
        return EpPlan((expert // epr).to(torch.int32), (base[expert] + pos).to(torch.int32), recv_counts, n_pairs)

    # ------------------------------------------------------------------ push / pull
    def push(self, x: torch.Tensor, token: Optional[torch.Tensor], scale: Optional[torch.Tensor], plan: EpPlan) -> None:
        """Row ``x[token[j]]`` (· ``scale[j]``) → row ``plan.dest_row[j]`` of rank ``plan.dest_rank[j]``'s receive buffer; ends
        with the barrier after which every rank may read what it received."""
        if self.cuda:
            from ..ops._lib import check, lib, stream_ptr

            if x.dtype != _BF16 or (scale is not None and scale.dtype != _BF16):
                raise TypeError("expert-parallel exchange on CUDA moves bf16 rows")
            token = None if token is None else token.contiguous()
            xc = x if x.is_contiguous() else x.contiguous()
            check(lib().ttb_ep_push(xc.data_ptr(), None if token is None else token.data_ptr(), None if scale is None else scale.contiguous().data_ptr(),
                                    plan.dest_rank.data_ptr(), plan.dest_row.data_ptr(), self._recv.pointer_array(), self.world, plan.n_pairs, self.dim,
                                    self.capacity, stream_ptr()), "ep_push")
        else:
            rows = x if token is None else x.index_select(0, token)
            if scale is not None:
                rows = rows * scale.reshape(-1, 1)
            rows = rows.float()
            gathered = self._all_gather_var([rows, plan.dest_rank.float(), plan.dest_row.float()])
            for r_rows, r_rank, r_row in gathered:
                mine = (r_rank.long() == self.rank) & (r_row.long() < self.capacity)
                self._recv_cpu[r_row.long()[mine]] = r_rows[mine]
        self.barrier()

    def pull(self, plan: EpPlan, dtype: torch.dtype) -> torch.Tensor:
        """``out[j] = result buffer of rank dest_rank[j], row dest_row[j]`` → ``[pairs, dim]`` (after :meth:`publish_result`)."""
        if self.cuda:
            from ..ops._lib import check, lib, stream_ptr

            out = torch.empty(plan.n_pairs, self.dim, dtype=_BF16, device=self.device)
            check(lib().ttb_ep_pull(self._result.pointer_array(), self.world, plan.dest_rank.data_ptr(), plan.dest_row.data_ptr(), out.data_ptr(), plan.n_pairs,
                                    self.dim, self.capacity, stream_ptr()), "ep_pull")
            return out
        results = [r[0] for r in self._all_gather_var([self._result_cpu])]
        stacked = torch.stack(results)  # [world, capacity, dim]
        row = plan.dest_row.long()
        ok = row < self.capacity
        out = stacked[plan.dest_rank.long(), row.clamp(max=self.capacity - 1)]
        return (out * ok.reshape(-1, 1)).to(dtype)

    def _all_gather_var(self, tensors: List[torch.Tensor]) -> List[List[torch.Tensor]]:
        if self.world == 1:
            return [tensors]
        out: List[Optional[List[torch.Tensor]]] = [None] * self.world
        dist.all_gather_object(out, [t.detach() for t in tensors], group=self.group)
        return out  # type: ignore[return-value]


def _clip_counts(recv_counts: torch.Tensor, capacity: int) -> torch.Tensor:
    end = recv_counts.cumsum(0).clamp(max=capacity)
    return end - torch.cat([end.new_zeros(1), end[:-1]])


class _Dispatch(torch.autograd.Function):
    """Routed rows to their experts' ranks.  Backward pulls the rows' gradients back and splits them into the token and
    score gradients (scores multiply the expert *input*, the Llama-4 convention)."""

    @staticmethod
    def forward(ctx, flat, scores, token_idx, plan: EpPlan, ep: ExpertParallelContext):
        ep.push(flat, token_idx, scores, plan)
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(flat, scores, token_idx)
        return ep.recv_rows(flat.dtype)

    @staticmethod
    def backward(ctx, d_recv):
        flat, scores, token_idx = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        ep.publish_result(d_recv)
        g = ep.pull(plan, flat.dtype)  # gradient w.r.t. each pushed row
        d_flat = d_scores = None
        if ctx.needs_input_grad[0]:
            d_flat = torch.zeros_like(flat).index_add_(0, token_idx, g * scores.reshape(-1, 1))
        if ctx.needs_input_grad[1]:
            d_scores = (flat.index_select(0, token_idx).float() * g.float()).sum(-1).to(scores.dtype)
        return d_flat, d_scores, None, None, None


class _Combine(torch.autograd.Function):
    """Expert outputs back to the ranks that own the tokens (one row per routed pair)."""

    @staticmethod
    def forward(ctx, y_local, plan: EpPlan, ep: ExpertParallelContext):
        ctx.ep, ctx.plan, ctx.rows = ep, plan, y_local.shape[0]
        ep.publish_result(y_local)
        return ep.pull(plan, y_local.dtype)

    @staticmethod
    def backward(ctx, d_pulled):
        ep, plan = ctx.ep, ctx.plan
        ep.push(d_pulled.contiguous(), None, None, plan)
        return ep.recv_rows(d_pulled.dtype)[: ctx.rows], None, None


class ExpertParallelMoE(nn.Module):
    """Drop-in replacement for :class:`torchtune_b200.modules.moe.MoE` that keeps ``num_experts / world`` experts per rank.
    Router and shared expert are replicated (their gradients are summed over the group before the optimizer step)."""

    def __init__(self, moe: nn.Module, ep: ExpertParallelContext):
        super().__init__()
        from ..modules.moe import GroupedExperts

        self.ep = ep
        self.router, self.shared_expert = moe.router, moe.shared_expert
        src = moe.experts
        if not isinstance(src, GroupedExperts):
            raise NotImplementedError("expert parallelism is implemented for GroupedExperts (full fine-tuning)")
        e0, e1 = ep.rank * ep.experts_per_rank, (ep.rank + 1) * ep.experts_per_rank
        local = GroupedExperts(dim=src.dim, hidden_dim=src.hidden_dim, num_experts=ep.experts_per_rank, activation=src.act_fn)
        for name in ("gate_proj", "up_proj", "down_proj"):
            w = getattr(src, name)
            setattr(local, name, nn.Parameter(w.detach()[e0:e1].clone(), requires_grad=w.requires_grad))
        self.experts = local

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bs, slen, dim = x.shape
        flat = x.reshape(bs * slen, dim)
        top_scores, token_indices, counts = self.router(flat)
        plan = self.ep.plan(counts, token_indices.numel())
        recv = _Dispatch.apply(flat, top_scores, token_indices, plan, self.ep)
        y_local = self.experts(recv, plan.recv_counts)
        pulled = _Combine.apply(y_local, plan, self.ep)
        out = self.shared_expert(flat) if self.shared_expert is not None else torch.zeros_like(flat)
        out = out.index_add(0, token_indices, pulled.to(out.dtype))
        return out.reshape(bs, slen, dim)

    def gather_full_experts(self) -> Dict[str, torch.Tensor]:
        """``{gate_proj, up_proj, down_proj}`` with all experts (collective)."""
        out = {}
        for name in ("gate_proj", "up_proj", "down_proj"):
            w = getattr(self.experts, name).detach()
            if self.ep.world == 1:
                out[name] = w
                continue
            src = w.float() if w.device.type == "cpu" and w.dtype == _BF16 else w
            parts = [torch.empty_like(src) for _ in range(self.ep.world)]
            dist.all_gather(parts, src.contiguous(), group=self.ep.group)
            out[name] = torch.cat(parts).to(w.dtype)
        return out


# ------------------------------------------------------------------------------------------- model level
def expert_parallelize(model: nn.Module, ep: ExpertParallelContext, replica_group=None, replicas: int = 1, prepare_layer=None) -> nn.Module:
    """Replace every :class:`MoE` layer of ``model`` by :class:`ExpertParallelMoE` (in place) and attach the small surface the
    sharded-model optimizer needs: ``_replicated`` (parameters every rank holds), ``sync_replicated_grads()`` and
    ``full_state_dict()`` (checkpoint layout with all experts; collective).

    When the expert-parallel group is smaller than the job (``replicas`` expert-parallel groups side by side), ``replica_group``
    holds the ranks that own the *same* experts: expert gradients are summed over it, dense gradients over every rank."""
    from ..modules.moe import MoE

    def swap(parent: nn.Module) -> None:
        for name, child in list(parent.named_children()):
            if isinstance(child, MoE):
                setattr(parent, name, ExpertParallelMoE(child, ep))
            else:
                swap(child)

    if prepare_layer is not None and hasattr(model, "layers"):
        # a model still on the meta device: every decoder layer gets storage and values (``prepare_layer(module, prefix)``, e.g.
        # training.LayerwisePreparer) right before its experts are cut down to this rank's, so the full expert stacks of at most
        # one layer are alive at a time
        import gc

        for i, layer in enumerate(model.layers):
            prepare_layer(layer, f"layers.{i}.")
            swap(layer)
            # the replaced MoE module (with the full expert stacks of this layer, 4 GB for a Scout layer) can sit in a reference
            # cycle; without a collection here the stacks of all layers pile up until the allocator runs out
            gc.collect()
        for name, child in model.named_children():
            if name != "layers":
                prepare_layer(child, f"{name}.")
    swap(model)
    expert_params = {id(p) for m in model.modules() if isinstance(m, ExpertParallelMoE) for p in m.experts.parameters()}
    model._replicated = [p for p in model.parameters() if id(p) not in expert_params]
    model._ep = ep

    def _sum(grads, group) -> None:
        big = [g for g in grads if g.numel() >= (1 << 20) and g.is_cuda and g.is_contiguous()]
        for g in big:  # large tensors are reduced in place; the many small ones share one flat fp32 buffer
            dist.all_reduce(g, group=group)
        grads = [g for g in grads if not any(g is b for b in big)]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=group)
        off = 0
        for g in grads:
            g.copy_(flat[off : off + g.numel()].view_as(g))
            off += g.numel()

    def sync_replicated_grads() -> None:
        if ep.world * replicas == 1:
            return
        # every rank trains on its own batch: dense parameters sum over the whole job (the default group when there are
        # several expert-parallel groups), experts over the ranks that hold the same ones
        _sum([p.grad for p in model._replicated if p.grad is not None], ep.group if replicas == 1 else None)
        if replicas > 1:
            _sum([p.grad for p in model.parameters() if id(p) in expert_params and p.grad is not None], replica_group)

    def full_state_dict() -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        gathered = {id(m): (name, m.gather_full_experts()) for name, m in model.named_modules() if isinstance(m, ExpertParallelMoE)}
        skip = {f"{name}.experts.{k}" for name, _ in gathered.values() for k in ("gate_proj", "up_proj", "down_proj")}
        for k, v in model.state_dict().items():
            if k not in skip:
                out[k] = v.detach()
        for name, full in gathered.values():
            for k, v in full.items():
                out[f"{name}.experts.{k}"] = v
        return out

    model.sync_replicated_grads = sync_replicated_grads
    model.full_state_dict = full_state_dict
    return model
