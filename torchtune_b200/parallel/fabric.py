"""Peer-memory fabric: device buffers that every rank of a process group can address.

A :class:`PeerBuffer` is allocated with ``cudaMalloc`` inside the kernel library, exported as
a CUDA IPC handle, exchanged once through ``torch.distributed`` and mapped by every rank, so
kernels receive a table of ``world`` base pointers and move data over NVLink with plain
loads/stores.  The reference has no counterpart (its collectives are NCCL calls made by
FSDP2/DTensor, torchtune/training/_distributed.py:661-714).
"""
from __future__ import annotations

import ctypes
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


class PeerBuffer:
    def __init__(self, nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.nbytes = int(nbytes)
        self.device = device
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
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
        if L.ttb_ipc_alloc(self.nbytes, ctypes.byref(out)) != 0 or not out.value:
            raise KernelError(f"cudaMalloc of {self.nbytes} bytes for a peer buffer failed")
        self.local_ptr = out.value
        self._local = torch.as_tensor(_RawCudaMemory(self.local_ptr, self.nbytes), device=device)
        self._local.zero_()
        self.peer_ptrs = [self.local_ptr]
        if self.world > 1:
            handle = ctypes.create_string_buffer(64)
            if L.ttb_ipc_get_handle(self.local_ptr, handle) != 0:
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
                self.peer_ptrs.append(p.value)
            torch.cuda.synchronize(device)
            dist.barrier(group=group)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        t = self._local[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def pointer_array(self):
        arr = (ctypes.c_void_p * len(self.peer_ptrs))(*self.peer_ptrs)
        return arr

    def close(self) -> None:
        if self.device.type != "cuda":
            return
        L = lib()
        for p in self._opened:
            L.ttb_ipc_close(p)
        self._opened = []
        if self.local_ptr:
            self._local = None
            L.ttb_ipc_free(self.local_ptr)
            self.local_ptr = 0
