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


class _PeerExchange:
    """The exchange as a push over peer memory: every rank writes its slices straight into the peers' receive buffers in their final
    layout (one kernel, ``ttb_cp_exchange``), with two flags per peer ordering it — "your previous data has been copied out of my
    buffer" before the push, "my data has arrived" after it (stores with release, bounded waits with acquire; no collective library).
    The result is copied out of the receive buffer because attention keeps q, k, v for its backward pass."""

    DATA, FREE = 0, 1

    def __init__(self, group, world: int, rank: int, device: torch.device):
        import ctypes

        from ..ops._lib import lib
        from .dp import _declare_dp
        from .fabric import PeerBuffer

        self.group, self.world, self.rank, self.device = group, world, rank, device
        self.L = lib()
        _declare_dp(self.L)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        self.L.ttb_cp_exchange.argtypes = [vp, ctypes.POINTER(vp), i32, i32, i32, i64, i64, i64, i64, vp]
        self.L.ttb_cp_exchange.restype = i32
        self.flags = PeerBuffer(world * self.L.ttb_dp_max_buckets() * 4, device, group)  # int32 [world][slots], zero-filled before the peers can see it
        self.recv = None
        self.epoch = 0
        self._PeerBuffer = PeerBuffer

    def _ensure(self, nbytes: int) -> None:
        if self.recv is not None and self.recv.nbytes >= nbytes:
            return
        if self.recv is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # nobody may still be pushing into the buffer that is about to be replaced
            self.recv.close()
        self.recv = self._PeerBuffer(max(nbytes, 1 << 20), self.device, self.group)

    def run(self, x: torch.Tensor, mode: int, out_shape, b: int, s_l: int, h_l: int, d: int) -> torch.Tensor:
        from ..ops._lib import check, err_word, stream_ptr

        x = x.contiguous()
        self._ensure(x.numel() * x.element_size())
        L, w = self.L, self.world
        err = err_word(self.device).data_ptr()
        self.epoch += 1
        if self.epoch > 1:  # every peer has copied the previous exchange out of its receive buffer
            check(L.ttb_dp_wait(self.flags.local_ptr, w, self.rank, self.FREE, self.epoch - 1, err, stream_ptr()), "cp wait (buffers free)")
        dv = d * x.element_size() // 16
        check(L.ttb_cp_exchange(x.data_ptr(), self.recv.pointer_array(), w, self.rank, mode, b, s_l, h_l, dv, stream_ptr()), "cp_exchange")
        check(L.ttb_dp_signal(self.flags.pointer_array(), w, self.rank, self.DATA, self.epoch, stream_ptr()), "cp signal (data)")
        check(L.ttb_dp_wait(self.flags.local_ptr, w, self.rank, self.DATA, self.epoch, err, stream_ptr()), "cp wait (data)")
        n = 1
        for k in out_shape:
            n *= k
        out = self.recv.tensor(x.dtype, n).view(out_shape).clone()
        check(L.ttb_dp_signal(self.flags.pointer_array(), w, self.rank, self.FREE, self.epoch, stream_ptr()), "cp signal (buffer free)")
        return out

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.recv is not None:
            self.recv.close()
            self.recv = None
        self.flags.close()


class ContextParallelContext:
    def __init__(self, group=None, *, world: Optional[int] = None, rank: Optional[int] = None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self._peer: Optional[_PeerExchange] = None

    def _peer_exchange(self, x: torch.Tensor) -> Optional[_PeerExchange]:
        """The peer-memory exchange for bf16 / fp16 CUDA tensors whose head dim fills whole 16-byte vectors (``TTB_CP_PEER=0`` keeps the
        collective-library all-to-all)."""
        import os

        if not (x.is_cuda and x.element_size() == 2 and (x.shape[-1] * 2) % 16 == 0 and self.world > 1 and os.environ.get("TTB_CP_PEER", "1") != "0"):
            return None
        if self._peer is None:
            self._peer = _PeerExchange(self.group, self.world, self.rank, x.device)
        return self._peer

    def shutdown(self) -> None:
        if self._peer is not None:
            self._peer.close()
            self._peer = None

    # raw exchanges ---------------------------------------------------------------------
    def _seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        b, s_l, h, d = x.shape
        w = self.world
        peer = self._peer_exchange(x)
        if peer is not None:
            return peer.run(x, 0, (b, w * s_l, h // w, d), b, s_l, h // w, d)
        send = x.reshape(b, s_l, w, h // w, d).permute(2, 0, 1, 3, 4).contiguous()
        recv = _all_to_all(send, self.group)  # [src rank = sequence block, b, s_l, h/w, d]
        return recv.permute(1, 0, 2, 3, 4).reshape(b, w * s_l, h // w, d)

    def _heads_to_seq(self, x: torch.Tensor) -> torch.Tensor:
        b, s, h_l, d = x.shape
        w = self.world
        peer = self._peer_exchange(x)
        if peer is not None:
            return peer.run(x, 1, (b, s // w, w * h_l, d), b, s // w, h_l, d)
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
