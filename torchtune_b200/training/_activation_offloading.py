"""Activation offloading to pinned host memory on a side stream.

Parity: torchtune/training/_activation_offloading.py:24-465.  Saved-for-backward tensors
of at least ``min_offload_size`` bytes that are neither parameters nor buffers are copied
device→host with ``cudaMemcpyAsync`` (``Tensor.copy_(non_blocking=True)`` into pinned
memory) on a dedicated copy stream while forward keeps running; backward brings each one
back on the same stream just before its consumer needs it.  Host buffers come from a
size-bucketed pinned pool that is reused across steps, so steady-state steps perform no
``cudaHostAlloc``.

Design differences from the reference: an explicit pinned pool, one event per transfer
(instead of stream-wide waits), and prefetch of the next ``prefetch`` tensors in backward
order when a tensor is unpacked.
"""
from __future__ import annotations

import contextlib
from collections import defaultdict
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn
from torch.autograd.graph import saved_tensors_hooks

from ..utils import get_logger

log = get_logger("DEBUG")


class PinnedPool:
    """Free lists of pinned host tensors keyed by (dtype, numel rounded up to 64 KiB)."""

    GRANULE = 64 * 1024

    def __init__(self) -> None:
        self._free: Dict[Tuple[torch.dtype, int], List[torch.Tensor]] = defaultdict(list)
        self.bytes_allocated = 0

    def _key(self, t: torch.Tensor) -> Tuple[torch.dtype, int]:
        nbytes = t.numel() * t.element_size()
        rounded = -(-nbytes // self.GRANULE) * self.GRANULE
        return t.dtype, rounded // t.element_size()

    def take(self, like: torch.Tensor) -> torch.Tensor:
        key = self._key(like)
        bucket = self._free[key]
        if bucket:
            return bucket.pop()
        self.bytes_allocated += key[1] * like.element_size()
        return torch.empty(key[1], dtype=like.dtype, pin_memory=True)

    def give(self, host: torch.Tensor) -> None:
        self._free[(host.dtype, host.numel())].append(host)


class _Slot:
    __slots__ = ("host", "shape", "stride", "device", "dtype", "d2h_done", "gpu", "h2d_done", "keepalive")

    def __init__(self) -> None:
        self.gpu: Optional[torch.Tensor] = None
        self.h2d_done: Optional[torch.cuda.Event] = None
        self.keepalive: Optional[torch.Tensor] = None


class OffloadActivations(saved_tensors_hooks):
    """Context manager; wrap the forward pass with it.

    Args:
        use_pin_memory: stage through pinned host memory (required for async copies).
        use_streams: run copies on a side stream overlapping compute; when False copies
            are issued on the compute stream (needed when other side streams interfere).
        max_fwd_stash_size: how many in-flight device→host copies may keep their source
            tensor alive before forward waits for the oldest one.
        min_offload_size: tensors smaller than this many bytes stay on the device.
        prefetch: how many upcoming tensors to bring back ahead of use in backward.
    """

    def __init__(
        self,
        use_pin_memory: bool = True,
        use_streams: bool = True,
        max_fwd_stash_size: int = 5,
        min_offload_size: int = 1024,
        virtual_memory_safe_pct: float = 60.0,
        prefetch: int = 2,
    ) -> None:
        self.use_pin_memory = use_pin_memory
        self.use_streams = use_streams and torch.cuda.is_available()
        self.max_fwd_stash_size = max_fwd_stash_size
        self.min_offload_size = min_offload_size
        self.virtual_memory_safe_pct = virtual_memory_safe_pct
        self.prefetch = prefetch
        self.pool = PinnedPool()
        self._copy_stream = torch.cuda.Stream() if self.use_streams else None
        self._slots: Dict[int, _Slot] = {}
        self._order: List[int] = []
        self._next_id = 0
        self._inflight: List[int] = []
        self._in_forward = True
        self._ignore: set = set()
        super().__init__(self._pack, self._unpack)

    # tensors that must stay on device (parameters, buffers) --------------------
    def register_resident(self, model: nn.Module) -> None:
        for t in list(model.parameters()) + list(model.buffers()):
            self._ignore.add(t.untyped_storage().data_ptr())

    def _host_memory_check(self) -> None:
        try:
            import psutil

            used = psutil.virtual_memory().percent
            if used > self.virtual_memory_safe_pct:
                log.warning(f"***** WARNING: host memory usage {used}% exceeds the safe threshold of {self.virtual_memory_safe_pct}% while offloading activations *****")
        except ImportError:
            pass

    def _pack(self, t: torch.Tensor) -> Any:
        if not self._in_forward_now():
            self._begin_forward()
        nbytes = t.numel() * t.element_size()
        if (
            not t.is_cuda
            or nbytes < self.min_offload_size
            or isinstance(t, nn.Parameter)
            or t.untyped_storage().data_ptr() in self._ignore
            or not t.is_contiguous()
        ):
            return t
        sid = self._next_id
        self._next_id += 1
        slot = _Slot()
        slot.shape, slot.stride, slot.device, slot.dtype = t.shape, t.stride(), t.device, t.dtype
        slot.host = self.pool.take(t) if self.use_pin_memory else torch.empty(t.numel(), dtype=t.dtype)
        compute = torch.cuda.current_stream()
        stream = self._copy_stream or compute
        if self._copy_stream is not None:
            self._copy_stream.wait_stream(compute)
        with torch.cuda.stream(stream):
            slot.host[: t.numel()].copy_(t.reshape(-1), non_blocking=True)
            slot.d2h_done = torch.cuda.Event()
            slot.d2h_done.record(stream)
        slot.keepalive = t  # keep the source alive until its copy has finished
        self._slots[sid] = slot
        self._order.append(sid)
        self._inflight.append(sid)
        while len(self._inflight) > self.max_fwd_stash_size:
            old = self._slots[self._inflight.pop(0)]
            old.d2h_done.synchronize()
            old.keepalive = None
        return ("offloaded", sid)

    def _in_forward_now(self) -> bool:
        return self._in_forward

    def _begin_forward(self) -> None:
        # first pack after a backward: recycle everything from the previous step
        for sid, slot in self._slots.items():
            if slot.host is not None and self.use_pin_memory:
                self.pool.give(slot.host)
        self._slots.clear()
        self._order.clear()
        self._inflight.clear()
        self._in_forward = True
        self._host_memory_check()

    def _issue_h2d(self, sid: int) -> None:
        slot = self._slots.get(sid)
        if slot is None or slot.gpu is not None:
            return
        compute = torch.cuda.current_stream()
        stream = self._copy_stream or compute
        slot.d2h_done.synchronize() if slot.keepalive is not None else None
        slot.keepalive = None
        with torch.cuda.stream(stream):
            if self._copy_stream is not None:
                stream.wait_event(slot.d2h_done)
            n = 1
            for d in slot.shape:
                n *= d
            gpu = torch.empty(n, dtype=slot.dtype, device=slot.device)
            gpu.copy_(slot.host[:n], non_blocking=True)
            slot.gpu = gpu.view(slot.shape)
            slot.h2d_done = torch.cuda.Event()
            slot.h2d_done.record(stream)

    def _unpack(self, packed: Any) -> torch.Tensor:
        if isinstance(packed, torch.Tensor):
            return packed
        self._in_forward = False
        _, sid = packed
        slot = self._slots[sid]
        self._issue_h2d(sid)
        # prefetch tensors saved just before this one (backward walks the order in reverse)
        pos = self._order.index(sid) if sid in self._order else -1
        for k in range(1, self.prefetch + 1):
            if pos - k >= 0:
                self._issue_h2d(self._order[pos - k])
        compute = torch.cuda.current_stream()
        compute.wait_event(slot.h2d_done)
        out = slot.gpu
        if self._copy_stream is not None:
            out.record_stream(compute)
        slot.gpu = None  # a second unpack (e.g. double backward) re-fetches
        return out


class NoOpManager(saved_tensors_hooks):
    """Inner context that disables an enclosing :class:`OffloadActivations` for a region
    (used around the output projection, whose large activation is consumed immediately)."""

    def __init__(self) -> None:
        super().__init__(lambda t: t, lambda t: t)


def get_act_offloading_ctx_manager(model: nn.Module, enable_activation_offloading: bool, use_streams: bool = True):
    """Return the context to wrap forward passes with.  When enabled, the model's output
    projection is exempted via forward hooks entering a :class:`NoOpManager`."""
    if not enable_activation_offloading:
        return contextlib.nullcontext()
    ctx = OffloadActivations(use_streams=use_streams)
    ctx.register_resident(model)
    noop = NoOpManager()
    output_head = None
    if hasattr(model, "output"):
        output_head = model.output
    elif hasattr(model, "decoder") and hasattr(model.decoder, "output"):
        output_head = model.decoder.output
    if output_head is None:
        raise ValueError("Activation offloading needs a model with an `output` projection (fusion models are not supported).")
    target = output_head if isinstance(output_head, nn.Module) else getattr(output_head, "linear", None)
    if isinstance(target, nn.Module):
        target.register_forward_pre_hook(lambda *a: noop.__enter__())
        target.register_forward_hook(lambda *a: noop.__exit__(None, None, None), always_call=True)
    return ctx
