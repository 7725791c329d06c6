"""Tensor parallelism with sequence-parallel activations over NVLink peer memory.

The reference builds tensor parallelism from DTensor plans (ColwiseParallel / RowwiseParallel /
SequenceParallel, torchtune/models/llama3/_parallelism.py:19-130) whose collectives are separate NCCL
kernels around cuBLAS GEMMs.  Here the two collective+GEMM pairs of a transformer block are single
kernels (``ttb_gemm_ag_bf16`` / ``ttb_gemm_rs_bf16`` in ``ops/csrc/gemm.cu``):

* column-parallel projection of a sequence-sharded input — *all-gather → GEMM*: extra copier warps inside the
  tcgen05 GEMM pull the peers' shards into local memory piece by piece (each byte crosses NVLink once) while the
  MMA pipeline works on the tiles that are already local; the TMA producer waits per m-tile on a piece counter;
* row-parallel projection to a sequence-sharded output — *GEMM → reduce-scatter*: the epilogue stores every
  output tile into a staging slot on the rank that owns those rows; the owner sums its ``world`` slots in fp32
  and adds the residual in the same pass.

Ordering between ranks uses readiness flags in peer memory instead of collectives: a one-warp kernel stores the
operation's epoch into every peer's flag array once this rank's shard (or its partial output tiles) is in place,
and the consuming kernel waits for the flags it needs with a cycle budget.  Shard and staging buffers are
double-buffered: a buffer is rewritten two operations later, and finishing the operation in between required
every peer's flag for it, which a peer stores only after its kernel that read the older buffer has completed.

Without CUDA (gloo) the same functions run on ``all_gather`` / ``reduce_scatter`` so the host-side logic is
testable on CPU.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .fabric import PeerBuffer

_BF16 = torch.bfloat16


def _declare(L) -> None:
    if getattr(L, "_tp_declared", False):
        return
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    pvp = ctypes.POINTER(vp)
    L.ttb_gemm_ag_bf16.argtypes = [pvp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i64, i64, vp, vp, i32, i32, i32, vp, vp]
    L.ttb_gemm_rs_bf16.argtypes = [vp, vp, pvp, i32, i32, i32, i32, i32, i32, i64, i64, i64, vp, vp]
    L.ttb_rs_reduce.argtypes = [vp, vp, vp, vp, i32, i64, i32, i64, i64, i64, vp, i32, i32, i32, i32, vp, vp]
    L.ttb_dp_signal.argtypes = [pvp, i32, i32, i32, i32, vp]
    L.ttb_dp_signal.restype = i32
    L.ttb_dp_max_buckets.restype = i32
    for fn in (L.ttb_gemm_ag_bf16, L.ttb_gemm_rs_bf16, L.ttb_rs_reduce):
        fn.restype = i32
    L._tp_declared = True


class TensorParallelContext:
    """Peer buffers and collective GEMMs for one tensor-parallel group.

    ``max_rows_per_rank`` is the largest number of tokens a rank owns (batch·seq / world) and
    ``max_width`` the widest activation that is gathered or scattered (the model width)."""

    def __init__(self, device: torch.device, group=None, *, max_rows_per_rank: int, max_width: int, keep_gathered: bool = True):
        self.device, self.group = device, group
        # keep the gathered activation a column-parallel layer's kernel produces for its weight gradient (saves one
        # all-gather per layer in backward at the price of holding world× the sharded activation until then)
        self.keep_gathered = keep_gathered
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.max_rows, self.max_width = int(max_rows_per_rank), int(max_width)
        self.cuda = device.type == "cuda"
        self._flip_g = 0
        self._flip_s = 0
        self._token = torch.zeros(1, device=device)
        if self.cuda:
            from ..ops._lib import lib

            _declare(lib())
            shard_bytes = self.max_rows * self.max_width * 2
            self._gather = [PeerBuffer(shard_bytes, device, group) for _ in range(2)]
            self._stage = [PeerBuffer(self.world * shard_bytes, device, group) for _ in range(2)]
            # readiness flags instead of collective barriers: slot 0/1 = gather buffers, 2/3 = staging buffers; a rank stores the
            # operation's epoch into every peer's array once its part is in place, consumers wait inside their kernels (bounded)
            self._flag_stride = lib().ttb_dp_max_buckets()
            self._flags = PeerBuffer(self.world * self._flag_stride * 4, device, group)
            self._epochs = [0, 0, 0, 0]

    # ------------------------------------------------------------------ plumbing
    def barrier(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def close(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            self.barrier()
            for b in self._gather + self._stage + [self._flags]:
                b.close()

    def _signal(self, slot: int) -> int:
        """Tell every peer that this rank's part of the operation using flag ``slot`` is in place (stream-ordered); returns the epoch
        the consumers wait for."""
        from ..ops._lib import check, lib, stream_ptr

        self._epochs[slot] += 1
        if self.world > 1:
            check(lib().ttb_dp_signal(self._flags.pointer_array(), self.world, self.rank, slot, self._epochs[slot], stream_ptr()), "tp_signal")
        return self._epochs[slot]

    def _check(self, rows: int, width: int) -> None:
        if rows > self.max_rows or width > self.max_width:
            raise ValueError(f"activation shard [{rows}, {width}] exceeds the context's buffers [{self.max_rows}, {self.max_width}]")

    @staticmethod
    def fusable(rows: int, k: int, n: int) -> bool:
        return rows % 128 == 0 and k % 8 == 0 and n % 8 == 0

    # ------------------------------------------------------------------ all-gather → GEMM
    def ag_gemm(self, x_shard: torch.Tensor, weight: torch.Tensor, *, b_mn: bool = False, bias: Optional[torch.Tensor] = None,
                return_gathered: bool = False):
        """``concat_ranks(x_shard) @ op(weight)`` → ``[world·rows, N]``; ``weight`` is ``[N, K]`` (or ``[K, N]`` with ``b_mn``).
        With ``return_gathered`` also returns ``concat_ranks(x_shard)`` — on the fused path it is a by-product of the kernel."""
        rows, k = x_shard.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        if not (self.cuda and x_shard.dtype == _BF16 and self.fusable(rows, k, n)):
            full = self.all_gather_rows(x_shard)
            out = full @ weight if b_mn else torch.nn.functional.linear(full, weight)
            out = out + bias if bias is not None else out
            return (out, full) if return_gathered else out
        from ..ops._lib import check, err_word, lib, stream_ptr

        self._check(rows, k)
        slot = self._flip_g
        buf = self._gather[slot]
        self._flip_g ^= 1
        buf.tensor(_BF16, rows * k).view(rows, k).copy_(x_shard)
        epoch = self._signal(slot)  # the copier warps of every peer wait for this flag before they read the shard
        out = torch.empty(self.world * rows, n, dtype=_BF16, device=self.device)
        gathered = torch.empty(self.world * rows, k, dtype=_BF16, device=self.device)
        sync = torch.empty(1 + self.world * rows // 128, dtype=torch.int32, device=self.device)
        w = weight if weight.is_contiguous() else weight.contiguous()
        check(
            lib().ttb_gemm_ag_bf16(buf.pointer_array(), w.data_ptr(), out.data_ptr(), gathered.data_ptr(), sync.data_ptr(), int(return_gathered),
                                   self.world, self.rank, rows, n, k, int(b_mn), w.stride(0), n,
                                   None if bias is None else bias.data_ptr(), self._flags.local_ptr if self.world > 1 else None, self._flag_stride, slot, epoch,
                                   err_word(self.device).data_ptr(), stream_ptr()),
            "gemm_ag",
        )
        return (out, gathered) if return_gathered else out

    # ------------------------------------------------------------------ GEMM → reduce-scatter
    def gemm_rs(self, x: torch.Tensor, weight: torch.Tensor, *, b_mn: bool = False, residual: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows ``[rank·rows, (rank+1)·rows)`` of ``Σ_ranks x_r @ op(weight_r)`` (+ residual, + bias) → ``[rows, N]``."""
        total, k = x.shape
        rows = total // self.world
        n = weight.shape[1] if b_mn else weight.shape[0]
        if not (self.cuda and x.dtype == _BF16 and total % self.world == 0 and self.fusable(rows, k, n)):
            partial = x @ weight if b_mn else torch.nn.functional.linear(x, weight)
            out = self.reduce_scatter_rows(partial)
            if residual is not None:
                out = out + residual
            return out + bias if bias is not None else out
        from ..ops._lib import check, err_word, lib, stream_ptr

        self._check(rows, n)
        slot = 2 + self._flip_s
        buf = self._stage[self._flip_s]
        self._flip_s ^= 1
        xc = x if x.is_contiguous() else x.contiguous()
        w = weight if weight.is_contiguous() else weight.contiguous()
        L = lib()
        check(L.ttb_gemm_rs_bf16(xc.data_ptr(), w.data_ptr(), buf.pointer_array(), self.world, self.rank, rows, n, k, int(b_mn), k, w.stride(0), n, err_word(self.device).data_ptr(), stream_ptr()), "gemm_rs")
        epoch = self._signal(slot)  # this rank's partial tiles have landed everywhere; the owner's sum waits for all peers' flags
        out = torch.empty(rows, n, dtype=_BF16, device=self.device)
        res = None if residual is None else (residual if residual.is_contiguous() else residual.contiguous())
        check(
            L.ttb_rs_reduce(buf.local_ptr, None if res is None else res.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), self.world, rows, n, n,
                            0 if res is None else res.stride(0), n, self._flags.local_ptr if self.world > 1 else None, self._flag_stride, slot, epoch, self.rank,
                            err_word(self.device).data_ptr(), stream_ptr()),
            "rs_reduce",
        )
        return out

    # ------------------------------------------------------------------ plain collectives (backward re-gathers, CPU path)
    def all_gather_rows(self, x_shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_shard
        out = torch.empty(self.world * x_shard.shape[0], *x_shard.shape[1:], dtype=x_shard.dtype, device=x_shard.device)
        src = x_shard.contiguous()
        if x_shard.device.type == "cpu" and x_shard.dtype == _BF16:
            parts = [torch.empty_like(src, dtype=torch.float32) for _ in range(self.world)]
            dist.all_gather(parts, src.float(), group=self.group)
            return torch.cat(parts).to(_BF16)
        dist.all_gather_into_tensor(out, src, group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        rows = x.shape[0] // self.world
        if x.device.type == "cpu":
            full = x.float().contiguous()
            dist.all_reduce(full, group=self.group)
            return full[self.rank * rows : (self.rank + 1) * rows].to(x.dtype)
        out = torch.empty(rows, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            if t.device.type == "cpu" and t.dtype == _BF16:
                f = t.float()
                dist.all_reduce(f, group=self.group)
                t.copy_(f)
            else:
                dist.all_reduce(t, group=self.group)
        return t


class _ColumnParallel(torch.autograd.Function):
    """``y[T, N_r] = gather(x_shard) · W_rᵀ``.  Backward: ``dx_shard = scatter-sum(dy · W_r)`` (fused GEMM → reduce-scatter),
    ``dW_r = dyᵀ · gather(x_shard)``."""

    @staticmethod
    def forward(ctx, x_shard, weight, tp: TensorParallelContext):
        ctx.tp = tp
        ctx.gathered = tp.keep_gathered and weight.requires_grad
        if ctx.gathered:  # the kernel's local copy of the gathered activation feeds the weight gradient; no re-gather
            out, x_full = tp.ag_gemm(x_shard, weight, return_gathered=True)
            ctx.save_for_backward(x_full, weight)
            return out
        ctx.save_for_backward(x_shard, weight)
        return tp.ag_gemm(x_shard, weight)

    @staticmethod
    def backward(ctx, dy):
        x_shard, weight = ctx.saved_tensors
        tp = ctx.tp
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = tp.gemm_rs(dy, weight, b_mn=True)
        if ctx.needs_input_grad[1]:
            x_full = x_shard if ctx.gathered else tp.all_gather_rows(x_shard)
            dw = _wgrad(dy, x_full, weight)
        return dx, dw, None


class _RowParallel(torch.autograd.Function):
    """``out_shard[rows, N] = scatter-sum(x[T, K_r] · W_rᵀ) (+ residual)``.  Backward: ``dx = gather(dy_shard) · W_r`` (fused
    all-gather → GEMM), ``dW_r = gather(dy_shard)ᵀ · x``; the residual receives ``dy_shard`` unchanged."""

    @staticmethod
    def forward(ctx, x, weight, residual, tp: TensorParallelContext):
        ctx.tp = tp
        ctx.has_residual = residual is not None
        ctx.save_for_backward(x, weight)
        return tp.gemm_rs(x, weight, residual=residual)

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        tp = ctx.tp
        dy_shard = dy_shard.contiguous()
        dx = dw = None
        dy_full = None
        if ctx.needs_input_grad[0]:
            if ctx.needs_input_grad[1]:
                dx, dy_full = tp.ag_gemm(dy_shard, weight, b_mn=True, return_gathered=True)
            else:
                dx = tp.ag_gemm(dy_shard, weight, b_mn=True)
        if ctx.needs_input_grad[1]:
            if dy_full is None:
                dy_full = tp.all_gather_rows(dy_shard)
            dw = _wgrad(dy_full, x, weight)
        return dx, dw, (dy_shard if ctx.has_residual and ctx.needs_input_grad[2] else None), None


def _wgrad(dy: torch.Tensor, x: torch.Tensor, weight: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``dyᵀ · x`` → ``[N, K]`` on the tcgen05 GEMM (TN form) when possible.  When ``weight`` lives in a flat parameter store the
    GEMM epilogue writes (or accumulates) straight into its window of the flat gradient buffer and ``None`` is returned."""
    if dy.is_cuda and dy.dtype == _BF16 and x.dtype == _BF16:
        from ..ops import _cuda
        from ..ops._cuda import gemm

        if weight is not None and _cuda.grad_window_owner(weight) is not None:
            return _cuda._wgrad(weight, dy if dy.is_contiguous() else dy.contiguous(), x if x.is_contiguous() else x.contiguous())
        return gemm(dy if dy.is_contiguous() else dy.contiguous(), x if x.is_contiguous() else x.contiguous(), a_mn=True, b_mn=True)
    return dy.t() @ x


def column_parallel_linear(x_shard: torch.Tensor, weight: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    return _ColumnParallel.apply(x_shard, weight, tp)


def row_parallel_linear(x: torch.Tensor, weight: torch.Tensor, tp: TensorParallelContext, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _RowParallel.apply(x, weight, residual, tp)
