"""Peer-memory fabric: device buffers that every rank of a process group can address.

A :class:`PeerBuffer` is allocated with ``cudaMalloc`` inside the kernel library, exported as
a CUDA IPC handle, exchanged once through ``torch.distributed`` and mapped by every rank, so
kernels receive a table of ``world`` base pointers and move data over NVLink with plain
loads/stores.  The reference has no counterpart (its collectives are NCCL calls made by
FSDP2/DTensor, torchtune/training/_distributed.py:661-714).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import KernelError, lib


class _RawCudaMemory:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view foreign device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def _declare(L) -> None:
    if getattr(L, "_fabric_declared", False):
        return
    vp, i64 = ctypes.c_void_p, ctypes.c_longlong
    L.ttb_ipc_alloc.argtypes = [i64, ctypes.POINTER(vp)]
    L.ttb_ipc_free.argtypes = [vp]
    L.ttb_ipc_get_handle.argtypes = [vp, ctypes.c_char_p]
    L.ttb_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.ttb_ipc_close.argtypes = [vp]
    L._fabric_declared = True


_GUARD_BYTE = 0xA5

# Pass as ``group`` to get a buffer that no peer maps (a store whose reduction group is this rank alone, e.g. the
# tensor-parallel shards when there is a single model replica) while the job has a default process group.
SOLO = object()


def _guard_bytes() -> int:
    """``TTB_PEER_GUARD_BYTES=<n>`` (debug aid, default 0) surrounds every peer buffer with ``n`` bytes (rounded up to 256) of a
    known pattern; :meth:`PeerBuffer.check_guards` then tells whether any kernel of any rank wrote outside the buffer."""
    n = int(os.environ.get("TTB_PEER_GUARD_BYTES", "0") or 0)
    return (n + 255) // 256 * 256 if n > 0 else 0


class PeerBuffer:
    # Device bytes held by live peer buffers of this process and their high-water mark.  These allocations bypass torch's
    # caching allocator, so ``torch.cuda.max_memory_allocated()`` does not see them; memory reports add ``peak_bytes``.
    live_bytes = 0
    peak_bytes = 0

    def __init__(self, nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.nbytes = int(nbytes)
        self.device = device
        self.guard = _guard_bytes() if device.type == "cuda" else 0
        self._base_ptr = 0
        self._whole: Optional[torch.Tensor] = None
        solo = group is SOLO or not dist.is_initialized()
        self.world = 1 if solo else dist.get_world_size(group)
        self.rank = 0 if solo else dist.get_rank(group)
        self._opened: List[int] = []
        if device.type != "cuda":
            # host stand-in used by the CPU (gloo) implementation of the same algorithms
            self._local = torch.zeros(self.nbytes, dtype=torch.uint8)
            self.local_ptr = self._local.data_ptr()
            self.peer_ptrs = [self.local_ptr]
            return
        L = lib()
        _declare(L)
        L.ttb_ensure_device(device.index if device.index is not None else torch.cuda.current_device())
        out = ctypes.c_void_p()
        g = self.guard
        if L.ttb_ipc_alloc(self.nbytes + 2 * g, ctypes.byref(out)) != 0 or not out.value:
            raise KernelError(f"cudaMalloc of {self.nbytes + 2 * g} bytes for a peer buffer failed")
        self._base_ptr = out.value
        self.local_ptr = out.value + g
        PeerBuffer.live_bytes += self.nbytes + 2 * g
        PeerBuffer.peak_bytes = max(PeerBuffer.peak_bytes, PeerBuffer.live_bytes)
        self._whole = torch.as_tensor(_RawCudaMemory(self._base_ptr, self.nbytes + 2 * g), device=device)
        self._local = self._whole[g : g + self.nbytes]
        self._local.zero_()
        if g:
            self._whole[:g].fill_(_GUARD_BYTE)
            self._whole[g + self.nbytes :].fill_(_GUARD_BYTE)
        self.peer_ptrs = [self.local_ptr]
        if self.world > 1:
            handle = ctypes.create_string_buffer(64)
            if L.ttb_ipc_get_handle(self._base_ptr, handle) != 0:
                raise KernelError("cudaIpcGetMemHandle failed")
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                p = ctypes.c_void_p()
                if L.ttb_ipc_open(h, ctypes.byref(p)) != 0 or not p.value:
                    raise KernelError(f"mapping the peer buffer of rank {r} failed (is peer access available?)")
                self._opened.append(p.value)
                self.peer_ptrs.append(p.value + g)  # every rank runs with the same guard size
            torch.cuda.synchronize(device)
            dist.barrier(group=group)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        t = self._local[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def check_guards(self) -> None:
        """Raise if the guard regions around this rank's buffer no longer hold their pattern (someone — a local kernel or a
        peer's — wrote outside the buffer).  No-op without ``TTB_PEER_GUARD_BYTES``."""
        if not self.guard or self._whole is None:
            return
        g = self.guard
        torch.cuda.synchronize(self.device)
        lo = int((self._whole[:g] != _GUARD_BYTE).sum().item())
        hi = int((self._whole[g + self.nbytes :] != _GUARD_BYTE).sum().item())
        if lo or hi:
            raise KernelError(f"peer buffer of {self.nbytes} bytes on rank {self.rank}: {lo} guard bytes below and {hi} above were overwritten")

    def pointer_array(self):
        arr = (ctypes.c_void_p * len(self.peer_ptrs))(*self.peer_ptrs)
        return arr

    def close(self) -> None:
        """Unmap the peers' buffers and free the own one; with guard regions enabled their pattern is verified first."""
        if self.device.type != "cuda":
            return
        L = lib()
        try:
            if self.local_ptr:
                self.check_guards()
        finally:
            for p in self._opened:
                L.ttb_ipc_close(p)
            self._opened = []
            if self.local_ptr:
                self._local = self._whole = None
                L.ttb_ipc_free(self._base_ptr)
                PeerBuffer.live_bytes -= self.nbytes + 2 * self.guard
                self.local_ptr = self._base_ptr = 0
