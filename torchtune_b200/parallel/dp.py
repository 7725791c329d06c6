"""Data parallelism with resident parameters and a sharded, fused optimizer step.

Design (sized for 180 GB of HBM per GPU): every rank keeps the full bf16 parameters and a
full bf16 gradient buffer as two *flat* peer-visible allocations; optimizer moments are
sharded.  The flat index space is cut into *buckets* (one per decoder layer, one for what
precedes the layers, one for what follows) and every rank owns the ``1 / world`` slice with
its rank's index of **every** bucket, so that the communication of one bucket keeps the
links of all GPUs busy.  The communication of a bucket is a single kernel per rank
(``ttb_dp_reduce_adamw_bcast``): pull the gradient slices of all peers, reduce in fp32,
AdamW on the owned slice, push the new parameters to all peers.  Buckets can be processed on a
side stream *during backward*, as soon as the layer's gradients are final on every rank
(a tensor hook on the layer's input gradient, a 4-byte all-reduce as the cross-rank
barrier), so reduction, optimizer and broadcast hide behind the backward GEMMs of the
earlier layers; with gradient clipping only the reduction is overlapped and the update
follows once the global norm is known.  (The hand-over during backward is opt-in through
``TTB_DP_OVERLAP_MIN_WORLD``; by default all buckets are processed right after backward.)  Compared with the reference's FSDP2 path
(per-layer all-gather in forward and backward, per-layer reduce-scatter, then a separate
scale pass and optimizer step — torchtune/training/_distributed.py:661-714,
recipes/full_finetune_distributed.py:1030-1050) this moves 2 instead of 3 model-sized
messages per step, keeps nothing on the critical path of the layers, and reduces in fp32
while sending bf16.

On CPU (gloo) the same interface is implemented with ``all_reduce`` so the host-side logic
is testable without GPUs.
"""
from __future__ import annotations

import ctypes
import math
import re
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from ..ops import reference as _ref
from .fabric import PeerBuffer

_LAYER_KEY = re.compile(r"^(.*\blayers\.\d+)\.")


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


def _bucket_key(name: str) -> Optional[str]:
    m = _LAYER_KEY.match(name)
    return m.group(1) if m else None


class FlatLayout:
    """Index arithmetic of a flat parameter space cut into buckets (no storage).

    ``buckets[b] = (start, size)`` are consecutive ranges of the flat index space whose sizes
    are multiples of ``8 · world``; rank ``r`` owns ``[start + r·size/world, start + (r+1)·size/world)``
    of each.  ``bucket_keys[b]`` is the module path of the decoder layer a bucket belongs to
    (``None`` for the parameters before / after the layers)."""

    def __init__(self, params: List[Tuple[str, nn.Parameter]], world: int, min_bucket_numel: int = 0):
        dtypes = {p.dtype for _, p in params}
        if len(dtypes) != 1:
            raise ValueError(f"all trainable parameters must share one dtype, found {dtypes}")
        self.dtype = dtypes.pop()
        self.world = world
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.offsets: List[int] = []
        self.buckets: List[Tuple[int, int]] = []
        self.bucket_keys: List[Optional[str]] = []
        self.bucket_params: List[List[nn.Parameter]] = []
        unit = 8 * world
        cursor, start, prev_key = 0, 0, object()
        for name, p in params:
            key = _bucket_key(name)
            if key != prev_key and self.bucket_params and cursor - start < min_bucket_numel:
                key = prev_key  # the running bucket is still small (e.g. only norm scales): the next layer joins it
            if key != prev_key and self.bucket_params:  # close the running bucket at a multiple of 8·world
                cursor = start + _round_up(cursor - start, unit)
                self.buckets.append((start, cursor - start))
                start = cursor
            if key != prev_key:
                self.bucket_keys.append(key)
                self.bucket_params.append([])
                prev_key = key
            self.offsets.append(cursor)
            self.bucket_params[-1].append(p)
            cursor += _round_up(p.numel(), 8)
        cursor = start + _round_up(max(cursor - start, unit), unit)
        self.buckets.append((start, cursor - start))
        self.total = cursor
        self.pieces = [size // world for _, size in self.buckets]
        self.state_offsets = [0]
        for piece in self.pieces:
            self.state_offsets.append(self.state_offsets[-1] + piece)
        self.shard = self.state_offsets[-1]  # elements of optimizer state per rank

    # ownership -----------------------------------------------------------------------------
    def owned(self, bucket: int, rank: int) -> Tuple[int, int, int]:
        """``(begin, count, state_offset)`` of rank ``rank``'s slice of ``bucket``."""
        start, _ = self.buckets[bucket]
        piece = self.pieces[bucket]
        return start + rank * piece, piece, self.state_offsets[bucket]

    def shards_to_full(self, shards: List[torch.Tensor]) -> torch.Tensor:
        """Per-rank state vectors (``[shard]`` each) → one vector in flat-parameter order (``[total]``)."""
        full = torch.zeros(self.total, dtype=shards[0].dtype, device=shards[0].device)
        for b in range(len(self.buckets)):
            for r, sh in enumerate(shards):
                begin, count, off = self.owned(b, r)
                full[begin : begin + count] = sh[off : off + count]
        return full

    def full_to_shard(self, full: torch.Tensor, rank: int, out: torch.Tensor) -> None:
        out.zero_()
        for b in range(len(self.buckets)):
            begin, count, off = self.owned(b, rank)
            end = min(begin + count, full.numel())
            if end > begin:
                out[off : off + end - begin].copy_(full[begin:end])


    # gradients -----------------------------------------------------------------------------
    def collect_autograd_grads(self, bucket: Optional[int] = None) -> None:
        """Move gradients that autograd produced as separate tensors into the flat buffer and
        zero the windows nothing wrote to (all parameters, or those of one bucket)."""
        for p in self.params if bucket is None else self.bucket_params[bucket]:
            if p.grad is not None:
                if p._grad_written:
                    p._grad_buffer.add_(p.grad)
                else:
                    p._grad_buffer.copy_(p.grad)
                p._grad_written = True
                p.grad = None
            elif not p._grad_written:
                p._grad_buffer.zero_()
                p._grad_written = True

    def reset_grad_flags(self) -> None:
        for p in self.params:
            p._grad_written = False


class FlatParameters(FlatLayout):
    """Re-homes the trainable parameters of ``model`` into one flat buffer (and gives each a
    same-shaped window of a flat gradient buffer, exposed as ``param._grad_buffer``); layout: :class:`FlatLayout`."""

    def __init__(self, params: List[Tuple[str, nn.Parameter]], world: int, device: torch.device, group=None, min_bucket_numel: int = 0):
        super().__init__(params, world, min_bucket_numel)
        esize = torch.empty(0, dtype=self.dtype).element_size()
        self.param_buf = PeerBuffer(self.total * esize, device, group)
        self.grad_buf = PeerBuffer(self.total * esize, device, group)
        self.flat_param = self.param_buf.tensor(self.dtype, self.total)
        self.flat_grad = self.grad_buf.tensor(self.dtype, self.total)
        with torch.no_grad():
            for p, off in zip(self.params, self.offsets):
                window = self.flat_param[off : off + p.numel()].view(p.shape)
                window.copy_(p.data)
                p.data = window
                p._grad_buffer = self.flat_grad[off : off + p.numel()].view(p.shape)
                p._grad_written = False
        if device.type == "cuda":
            from ..ops import _cuda

            for p in self.params:
                _cuda.register_grad_window(p)

    def close(self) -> None:
        self.param_buf.close()
        self.grad_buf.close()


class ShardedAdamW:
    """AdamW over a :class:`FlatParameters` store; this rank updates its slice of every bucket
    and the fused kernel distributes the result.  ``step`` handles all buckets that were not
    already processed during backward (:meth:`begin_step` / :meth:`process_bucket`)."""

    def __init__(self, flat: FlatParameters, rank: int, world: int, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, group=None):
        self.flat, self.rank, self.world, self.group = flat, rank, world, group
        self.param_groups = [dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, params=flat.params)]
        dev = flat.flat_param.device
        self.exp_avg = torch.zeros(flat.shard, dtype=flat.dtype, device=dev)
        self.exp_avg_sq = torch.zeros(flat.shard, dtype=flat.dtype, device=dev)
        self.step_count = 0
        self._gsum: Optional[torch.Tensor] = None
        self._partials: Optional[torch.Tensor] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._open: Optional[Dict[str, Any]] = None  # state of a step whose buckets are processed one by one

    # torch.optim-like surface used by schedulers / loggers
    @property
    def torch_optimizer(self):
        return self

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.reset_grad_flags()

    def state_dict(self) -> Dict[str, Any]:
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(saved)

    def full_state_dict(self, is_rank_zero: bool = True, group=None) -> Dict[str, Any]:
        """Moments of the whole model as one CPU tensor each, in flat-parameter order, plus the parameter
        layout, so a checkpoint written at one world size can be read at another."""
        flat = self.flat
        group = group if group is not None else self.group
        out = {}
        for key, shard in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            if self.world > 1:
                src = shard.float() if (shard.device.type == "cpu" and shard.dtype == torch.bfloat16) else shard  # gloo has no bf16 all_gather
                parts = [torch.empty_like(src) for _ in range(self.world)]
                dist.all_gather(parts, src, group=group)
                parts = [p.to(shard.dtype) for p in parts]
            else:
                parts = [shard]
            out[key] = flat.shards_to_full([p.cpu() for p in parts]) if is_rank_zero else None
        if not is_rank_zero:
            return {}
        out["step"] = self.step_count
        out["layout"] = {"names": list(flat.names), "offsets": list(flat.offsets), "numels": [p.numel() for p in flat.params]}
        out["param_groups"] = [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]
        return out

    def load_full_state_dict(self, sd: Dict[str, Any]) -> None:
        flat = self.flat
        layout = sd.get("layout")
        if layout is not None and (list(layout["names"]) != list(flat.names) or list(layout["numels"]) != [p.numel() for p in flat.params]):
            raise ValueError("optimizer checkpoint was written for a different set of trainable parameters")
        self.step_count = int(sd["step"])
        for key, shard in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            full = sd[key]
            if layout is not None and list(layout["offsets"]) != list(flat.offsets):
                # written with another world size (bucket padding differs): move every parameter's window
                moved = torch.zeros(flat.total, dtype=full.dtype)
                for old, new, n in zip(layout["offsets"], flat.offsets, layout["numels"]):
                    moved[new : new + n] = full[old : old + n]
                full = moved
            flat.full_to_shard(full, self.rank, shard)
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(saved)

    # ------------------------------------------------------------------ step protocol
    def begin_step(self, grad_scale: Union[float, torch.Tensor], max_grad_norm: Optional[float]) -> None:
        """Open a step whose buckets may be processed one at a time (:meth:`process_bucket`) before :meth:`step` finishes it."""
        g = self.param_groups[0]
        self.step_count += 1
        b1, b2 = g["betas"]
        st: Dict[str, Any] = dict(
            done=set(), clip=max_grad_norm, inv_bc1=1.0 / (1.0 - b1**self.step_count), inv_sqrt_bc2=1.0 / math.sqrt(1.0 - b2**self.step_count),
            scale_dev=None, scale_host=1.0,
        )
        if isinstance(grad_scale, torch.Tensor):
            st["scale_dev"] = grad_scale.detach().to(torch.float32).reshape(1)
        else:
            st["scale_host"] = float(grad_scale)
        flat = self.flat
        if max_grad_norm is not None and flat.flat_param.is_cuda:
            from ..ops._lib import lib

            if self._gsum is None:
                self._gsum = torch.empty(flat.shard, dtype=torch.float32, device=flat.flat_param.device)
            grid = lib().ttb_dp_grid()
            self._partials = torch.zeros(len(flat.buckets) * grid, dtype=torch.float32, device=flat.flat_param.device)
            st["grid"] = grid
        self._open = st

    def process_bucket(self, bucket: int) -> None:
        """CUDA only.  Without clipping: reduce + AdamW + broadcast of this bucket.  With clipping: reduce into the fp32
        scratch and accumulate the squared norm; the update follows in :meth:`step`."""
        st = self._open
        if st is None or bucket in st["done"]:
            return
        st["done"].add(bucket)
        if st["clip"] is None:
            self._launch(bucket, 0, st, st["scale_dev"], st["scale_host"])
        else:
            self._launch(bucket, 1, st, None, 1.0)

    def _launch(self, bucket: int, mode: int, st: Dict[str, Any], sdev, shost) -> None:
        from ..ops._lib import check, lib, stream_ptr

        L = lib()
        _declare_dp(L)
        flat, g = self.flat, self.param_groups[0]
        begin, count, off = flat.owned(bucket, self.rank)
        b1, b2 = g["betas"]
        esz = self.exp_avg.element_size()
        gsum = None if self._gsum is None or mode == 0 else self._gsum.data_ptr() + 4 * off
        partials = None if mode != 1 else self._partials.data_ptr() + 4 * bucket * st["grid"]
        from ..ops._lib import err_word

        wait = st.get("wait") if mode != 2 else None  # (local flag array, epoch): set while buckets are processed during backward
        check(
            L.ttb_dp_reduce_adamw_bcast(flat.grad_buf.pointer_array(), flat.param_buf.pointer_array(), self.world, self.rank, begin, count,
                                        self.exp_avg.data_ptr() + esz * off, self.exp_avg_sq.data_ptr() + esz * off, gsum, partials,
                                        None if sdev is None else sdev.data_ptr(), shost, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"],
                                        st["inv_bc1"], st["inv_sqrt_bc2"], mode, None if wait is None else wait[0], bucket, 0 if wait is None else wait[1],
                                        err_word(flat.flat_param.device).data_ptr(), int(st.get("grid_ctas", 0)) if mode != 2 else 0, 1, 0, stream_ptr()),
            "dp_reduce_adamw_bcast",
        )

    # The step in three collective-free pieces, so that several stores with different reduction groups can share one clipping
    # norm (:class:`~torchtune_b200.parallel.stores.MultiStoreAdamW`); :meth:`step` strings them together for a single store.
    def reduce_all(self, group=None) -> None:
        """Sum every bucket over the store's ranks.  Without clipping the CUDA kernels also update and broadcast here."""
        st = self._open
        if not self.flat.flat_param.is_cuda:
            self._host_reduce(st, group if group is not None else self.group)
            return
        for b in range(len(self.flat.buckets)):
            self.process_bucket(b)

    def local_sumsq(self) -> torch.Tensor:
        """Sum of squares of the reduced (unscaled) gradient over *this rank's* slices; summed over the store's ranks it is the
        squared norm of the whole store."""
        st = self._open
        if not self.flat.flat_param.is_cuda:
            return st["gsum"][st["mine"]].pow(2).sum()
        return self._partials.sum()

    def finish(self, total_sumsq: Optional[torch.Tensor]) -> None:
        """Apply the update; ``total_sumsq`` is the squared global gradient norm (required when the step clips)."""
        st = self._open
        self.last_grad_norm = None
        try:
            flat = self.flat
            if st["scale_dev"] is not None:
                s = st["scale_dev"].to(flat.flat_param.device)
            else:
                s = torch.tensor([st["scale_host"]], dtype=torch.float32, device=flat.flat_param.device)
            coef = None
            if st["clip"] is not None:
                norm = total_sumsq.to(torch.float32).sqrt() * s
                self.last_grad_norm = norm.reshape(())
                coef = (torch.clamp(float(st["clip"]) / (norm + 1e-6), max=1.0) * s).reshape(1).float()
            if not flat.flat_param.is_cuda:
                self._host_apply(st, float((coef if coef is not None else s).item()))
            elif coef is not None:
                for b in range(len(flat.buckets)):
                    self._launch(b, 2, st, coef, 1.0)
        finally:
            self._open = None

    def step(self, grad_scale: Union[float, torch.Tensor] = 1.0, max_grad_norm: Optional[float] = None, group=None) -> None:
        if self._open is None:
            self.begin_step(grad_scale, max_grad_norm)
        group = group if group is not None else self.group
        try:
            self.reduce_all(group)
            total = None
            if self._open["clip"] is not None:
                total = self.local_sumsq()
                if self.world > 1:
                    dist.all_reduce(total, group=group)
        except BaseException:
            self._open = None
            raise
        self.finish(total)

    def _host_reduce(self, st: Dict[str, Any], group) -> None:
        """gloo statement of the reduction: fp32 sum of all ranks' gradients; ``mine`` indexes this rank's slices."""
        flat = self.flat
        gsum = flat.flat_grad.float()
        if self.world > 1:
            dist.all_reduce(gsum, group=group)
        st["gsum"] = gsum
        st["mine"] = torch.cat([torch.arange(begin, begin + count) for begin, count, _ in (flat.owned(b, self.rank) for b in range(len(flat.buckets)))])
        st["group"] = group

    def _host_apply(self, st: Dict[str, Any], scale: float) -> None:
        """gloo statement of update + broadcast: AdamW on the owned slices, then every rank collects all slices."""
        flat, g = self.flat, self.param_groups[0]
        b1, b2 = g["betas"]
        mine = st["mine"]
        new = flat.flat_param[mine].clone()
        _ref.adamw_step(new, st["gsum"][mine], self.exp_avg, self.exp_avg_sq, self.step_count, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"], scale)
        if self.world > 1:
            gathered = [torch.empty_like(new) for _ in range(self.world)]
            if new.dtype == torch.bfloat16:  # gloo has no bf16 all_gather
                parts = [torch.empty(new.shape, dtype=torch.float32) for _ in range(self.world)]
                dist.all_gather(parts, new.float(), group=st["group"])
                gathered = [p.to(new.dtype) for p in parts]
            else:
                dist.all_gather(gathered, new, group=st["group"])
            flat.flat_param.copy_(flat.shards_to_full(gathered))
        else:
            flat.flat_param[mine] = new


def _declare_dp(L) -> None:
    if getattr(L, "_dp_declared", False):
        return
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    L.ttb_dp_reduce_adamw_bcast.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, i64, i64, vp, vp, vp, vp, vp, f32, f32, f32, f32, f32, f32, f32, f32, i32, vp, i32, i32, vp, i32, i32, i32, vp]
    L.ttb_dp_reduce_adamw_bcast.restype = i32
    L.ttb_dp_signal.argtypes = [ctypes.POINTER(vp), i32, i32, i32, i32, vp]
    L.ttb_dp_signal.restype = i32
    L.ttb_zero3_gather.argtypes = [ctypes.POINTER(vp), i32, i32, i64, vp, vp, i32, i32, vp, i32, vp]
    L.ttb_zero3_gather.restype = i32
    L.ttb_dp_wait.argtypes = [vp, i32, i32, i32, i32, vp, vp]
    L.ttb_dp_wait.restype = i32
    L.ttb_dp_grid.restype = i32
    L.ttb_dp_max_buckets.restype = i32
    L.ttb_dp_set_wait_cycles.argtypes = [i64]
    L.ttb_dp_set_wait_cycles.restype = None
    L._dp_declared = True


class DataParallelEngine:
    """Owns the flat stores, the wgrad side stream and the step protocol.

    Step protocol: ``arm_backward_overlap(optimizer, grad_scale, clip)`` → backward, during which every decoder layer's
    bucket is handed to the optimizer on the communication stream as soon as its gradients are final (hook on the
    gradient of the layer's input; a 4-byte all-reduce on that stream tells every rank the bucket is final everywhere)
    → ``optimizer_step`` processes what is left (embeddings, anything without a hook), joins the streams and closes with a
    small all-reduce (new parameters have landed everywhere and nobody still reads the old gradients).  Without arming,
    ``optimizer_step`` runs the whole protocol after backward.
    """

    def __init__(self, device: torch.device, group=None):
        self.device = device
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.flat: Optional[FlatParameters] = None
        self._barrier_token = torch.zeros(1, device=device if device.type == "cuda" else "cpu")
        self._bucket_token = torch.zeros(1, device=device if device.type == "cuda" else "cpu")
        self._comm_stream = None
        self._armed = None  # the optimizer whose buckets are processed during the running backward
        self._flags = None
        import os

        # Handing buckets to the optimizer during backward is opt-in (set the smallest world size it should be used at):
        # measured on the 8B model it lost on 1 and 2 GPUs (the HBM-bound update competes with the backward GEMMs) and
        # made no difference on 4 (≈ 484 ms per step either way), so the simpler after-backward protocol is the default.
        self.min_world_for_overlap = int(os.environ.get("TTB_DP_OVERLAP_MIN_WORLD", "1000000"))
        # CTAs of a bucket kernel that runs beside the backward GEMMs (NVLink-bound: a few dozen CTAs saturate the links and leave
        # HBM bandwidth and issue slots to the GEMMs); 0 = the full grid
        self.overlap_ctas = int(os.environ.get("TTB_DP_OVERLAP_CTAS", "0")) or max(48, 592 // max(self.world, 1))
        self._barrier_epoch = 0

    # sizes the recipes ask for ------------------------------------------------------------
    dp_size = property(lambda self: self.world)
    dp_rank = property(lambda self: self.rank)
    non_data_parallel_size = 1
    min_seq_len_divisor = 1

    def prepare(self, model: nn.Module) -> nn.Module:
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.flat = FlatParameters(named, self.world, self.device, self.group)
        if self.device.type == "cuda":
            from ..ops import _cuda

            _cuda.enable_direct_wgrad(True)
            from ..ops._lib import lib

            L = lib()
            _declare_dp(L)
            if len(self.flat.buckets) < L.ttb_dp_max_buckets():
                self._comm_stream = torch.cuda.Stream(device=self.device)
                self._flags = PeerBuffer(self.world * L.ttb_dp_max_buckets() * 4, self.device, self.group)  # int32 [world][max buckets]
                self._epoch = 0
                self._install_bucket_hooks(model)
        return model

    # ------------------------------------------------------------------ backward overlap
    def _install_bucket_hooks(self, model: nn.Module) -> None:
        """The gradient of a layer's input is complete only after every node of that layer has run, so a hook on it marks
        the layer's bucket as final; the gradient of the last layer's output does the same for what follows the layers."""
        keys = self.flat.bucket_keys
        last = None
        for b, key in enumerate(keys):
            if key is None:
                continue
            try:
                mod = model.get_submodule(key)
            except AttributeError:
                continue
            mod.register_forward_pre_hook(self._pre_hook(b))
            last = (b, mod)
        if last is not None and last[0] + 1 < len(keys) and keys[last[0] + 1] is None:
            last[1].register_forward_hook(self._post_hook(last[0] + 1))

    def _watch(self, t: Any, bucket: int) -> None:
        if self._armed is not None and torch.is_tensor(t) and t.requires_grad and torch.is_grad_enabled():
            t.register_hook(lambda g, b=bucket: self._bucket_ready(b))

    def _pre_hook(self, bucket: int):
        return lambda module, args: self._watch(args[0] if args else None, bucket)

    def _post_hook(self, bucket: int):
        def hook(module, args, output):
            self._watch(output[0] if isinstance(output, (tuple, list)) else output, bucket)

        return hook

    def wants_backward_overlap(self, optimizer) -> bool:
        """Whether :meth:`arm_backward_overlap` would arm: CUDA, a bucket-wise optimizer, and enough ranks for the hidden NVLink
        traffic to outweigh what the concurrent HBM-bound update costs the backward GEMMs (on one GPU nothing crosses NVLink and
        overlapping only took bandwidth and power from the GEMMs: 506 vs 488 ms per step on the 8B model; 530 vs 503 on two)."""
        return self._comm_stream is not None and hasattr(optimizer, "process_bucket") and self._armed is None and self.world >= self.min_world_for_overlap

    def arm_backward_overlap(self, optimizer, grad_scale, clip_grad_norm: Optional[float] = None) -> bool:
        """Call between the forward pass and ``backward()`` of the step's last micro-batch, with the final gradient scale."""
        if not self.wants_backward_overlap(optimizer):
            return False
        optimizer.begin_step(grad_scale, clip_grad_norm)
        self._epoch += 1
        optimizer._open["wait"] = (self._flags.local_ptr, self._epoch)
        optimizer._open["grid_ctas"] = self.overlap_ctas
        self._armed = optimizer
        return True

    def _bucket_ready(self, bucket: int) -> None:
        opt = self._armed
        if opt is None:
            return None
        self._hand_over([bucket], opt)
        return None

    def _hand_over(self, buckets: List[int], opt) -> None:
        from ..ops import _cuda

        for b in buckets:
            self.flat.collect_autograd_grads(b)
        main, comm = torch.cuda.current_stream(self.device), self._comm_stream
        comm.wait_stream(main)
        if _cuda._wgrad_stream is not None:
            comm.wait_stream(_cuda._wgrad_stream)
        from ..ops._lib import check, lib, stream_ptr

        with torch.cuda.stream(comm):
            for b in buckets:
                # tell every peer that this rank's gradients of bucket b are final; the bucket kernel waits for the peers' flags
                check(lib().ttb_dp_signal(self._flags.pointer_array(), self.world, self.rank, b, self._epoch, stream_ptr()), "dp_signal")
                opt.process_bucket(b)

    def build_optimizer(self, model: nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, **_: Any) -> ShardedAdamW:
        if self.flat is None:
            raise RuntimeError("call prepare(model) first")
        return ShardedAdamW(self.flat, self.rank, self.world, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def all_reduce_sum_(self, *tensors: torch.Tensor) -> None:
        if self.world == 1:
            return
        if len(tensors) == 1:
            dist.all_reduce(tensors[0], group=self.group)
            return
        packed = torch.stack([t.reshape(()).to(torch.float32) for t in tensors])
        dist.all_reduce(packed, group=self.group)
        for t, v in zip(tensors, packed):
            t.copy_(v)

    def barrier(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._barrier_token, group=self.group)

    def _step_barrier(self) -> None:
        """Stream-ordered barrier between the ranks on peer-memory flags (two one-warp kernels of the kernel library: store the
        epoch into every peer's flag array, then wait — bounded — until all peers' entries have arrived).  Everything this rank
        enqueued before is complete (and its peer stores visible) when a peer gets past its wait.  Falls back to a 4-byte
        all-reduce when the flag array does not exist (CPU, or more buckets than flag slots)."""
        if self.world == 1:
            return
        if self._flags is None:
            self.barrier()
            return
        from ..ops._lib import check, err_word, lib, stream_ptr

        L = lib()
        self._barrier_epoch += 1
        slot = L.ttb_dp_max_buckets() - 1  # the last slot is never a bucket's (prepare() keeps bucket counts below it)
        check(L.ttb_dp_signal(self._flags.pointer_array(), self.world, self.rank, slot, self._barrier_epoch, stream_ptr()), "dp_signal")
        check(L.ttb_dp_wait(self._flags.local_ptr, self.world, self.rank, slot, self._barrier_epoch, err_word(self.device).data_ptr(), stream_ptr()), "dp_wait")

    def optimizer_step(self, model: nn.Module, optimizer: ShardedAdamW, grad_scale, clip_grad_norm: Optional[float] = None):
        if self._armed is not None:
            if self._armed is not optimizer:
                raise RuntimeError("optimizer_step was called with another optimizer than the armed one")
            left = [b for b in range(len(self.flat.buckets)) if b not in optimizer._open["done"]]
            if left:
                self._hand_over(left, optimizer)
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
            self._armed = None
            optimizer.step(grad_scale=grad_scale, max_grad_norm=clip_grad_norm, group=self.group)  # with clipping: norm + update
            if self.world > 1:
                self._step_barrier()  # pushes have landed; gradients may be overwritten
            optimizer.zero_grad()
            return optimizer.last_grad_norm
        if self.device.type == "cuda":
            from ..ops import _cuda

            _cuda.join_wgrad_stream()
        self.flat.collect_autograd_grads()
        if self.world > 1 and self.device.type == "cuda":
            self._step_barrier()  # every rank's gradient buffer is complete
        optimizer.step(grad_scale=grad_scale, max_grad_norm=clip_grad_norm, group=self.group)
        if self.world > 1 and self.device.type == "cuda":
            self._step_barrier()  # pushes have landed; gradients may be overwritten
        optimizer.zero_grad()
        return optimizer.last_grad_norm

    def shutdown(self) -> None:
        if self.flat is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.barrier()
            if self._flags is not None:
                self._flags.close()
                self._flags = None
            self.flat.close()
            self.flat = None
