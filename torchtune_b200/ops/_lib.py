"""ctypes loader for the in-tree kernel library ``_lib/libttb200.so``.

The library is looked up next to this file; on a machine with a CUDA device a missing
library is a hard error (operators never fall back silently), on CPU-only machines the
loader is simply never invoked.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "_lib" / "libttb200.so"
_lib: Optional[ctypes.CDLL] = None
_err_words = {}

ERROR_NAMES = {-1: "bad shape or alignment", -2: "driver / launch failure", -3: "size beyond a static limit", -4: "device wait timed out"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise KernelError(
                f"{LIB_PATH} is missing. Build it with `python -m torchtune_b200.ops.build` (needs nvcc); "
                "CUDA tensors are never routed to a PyTorch fallback."
            )
        _lib = ctypes.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    c = ctypes
    vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    L.ttb_gemm_bf16.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, i32, vp, f32, vp, vp]
    L.ttb_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, i32, i32, f32, vp]
    L.ttb_rmsnorm_bwd_partials.argtypes = [i32]
    L.ttb_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, vp]
    L.ttb_rope.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, vp]
    L.ttb_kd_divergence.argtypes = [vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, i64, f32, f32, vp]
    L.ttb_kd_divergence.restype = i32
    L.ttb_sample.argtypes = [vp, i64, i32, vp, i64, vp, i32, i32, f32, i32, vp]
    L.ttb_sample.restype = i32
    L.ttb_index_violations.argtypes = [i32]
    L.ttb_index_violations.restype = ctypes.c_uint32
    L.ttb_swiglu_fwd.argtypes = [vp, vp, vp, i64, i32, i64, i64, i64, vp]
    L.ttb_swiglu_bwd.argtypes = [vp, vp, vp, vp, vp, i64, i32, i64, i64, i64, i64, i64, vp]
    L.ttb_adamw.argtypes = [vp, i32, i64, i32, f32, f32, f32, f32, f32, f32, f32, vp, f32, vp]
    L.ttb_adamw8bit.argtypes = [vp, vp, vp, vp, vp, vp, i64, i32, f32, f32, f32, f32, f32, f32, f32, vp, f32, vp]
    L.ttb_grad_sumsq.argtypes = [vp, i32, i64, i32, vp, vp]
    L.ttb_softmax_ce.argtypes = [vp, vp, vp, vp, i32, i32, i64, i64, i32, vp]
    L.ttb_softmax_ce_capped.argtypes = [vp, vp, vp, vp, i32, i32, i64, i64, i32, ctypes.c_float, vp]
    L.ttb_attn_fwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, f32, vp, vp]
    L.ttb_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, f32, vp, vp]
    L.ttb_attn_bwd.restype = i32
    L.ttb_attn_fwd.restype = i32
    L.ttb_attn_fwd2.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp, vp]
    L.ttb_attn_fwd2.restype = i32
    L.ttb_gemm_bf16_2sm.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, vp, f32, vp, vp]
    L.ttb_gemm_bf16_2sm.restype = i32
    L.ttb_ensure_device.argtypes = [i32]
    L.ttb_gemm_grouped_bf16.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i64, i64, i64, i64, vp, vp]
    L.ttb_gemm_grouped_bf16.restype = i32
    L.ttb_gemm_bf16_dual.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64, i32, i32, vp, f32, vp, vp]
    L.ttb_gemm_bf16_dual.restype = i32
    L.ttb_gemm_bf16_dual_2sm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64, vp, f32, vp, vp]
    L.ttb_gemm_bf16_dual_2sm.restype = i32
    L.ttb_gemm_bf16_2sm_residual.argtypes = [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, vp, vp, vp]
    L.ttb_gemm_bf16_2sm_residual.restype = i32
    L.ttb_gemm_bf16_splitk.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, f32, vp, vp]
    L.ttb_gemm_bf16_splitk.restype = i32
    L.ttb_gemm_grouped_wgrad_bf16.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i64, i64, i64, i64, i32, vp, vp]
    L.ttb_gemm_grouped_wgrad_bf16.restype = i32
    L.ttb_nf4_dequant.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, vp]
    L.ttb_nf4_dequant.restype = i32
    L.ttb_nf4_absmax.argtypes = [vp, vp, i64, i32, vp]
    L.ttb_nf4_encode.argtypes = [vp, vp, vp, i64, i32, vp]
    L.ttb_nf4_absmax.restype = i32
    L.ttb_nf4_encode.restype = i32
    L.ttb_moe_route_sort.argtypes = [vp, i32, i32, vp, vp, vp]
    L.ttb_moe_permute_indices.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.ttb_embedding_fwd.argtypes = [vp, vp, vp, i64, i32, i64, vp]
    L.ttb_embedding_bwd.argtypes = [vp, vp, vp, vp, i64, i32, i64, i64, vp]
    L.ttb_gemm_fp8.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, vp, i32, vp, i32, vp, i32, vp, vp]
    L.ttb_fp8_cast_transpose.argtypes = [vp, i64, i32, i32, vp, i32, vp, vp, i32, vp, i32, vp]
    L.ttb_gemm_fp8.restype = i32
    L.ttb_mx_scale_bytes.argtypes = [i64, i64]
    L.ttb_mx_scale_bytes.restype = i64
    L.ttb_mx_quantize.argtypes = [vp, i64, vp, i64, vp, i64, i64, i32, vp]
    L.ttb_mx_quantize.restype = i32
    L.ttb_mx_quantize_both.argtypes = [vp, i64, vp, i64, vp, vp, i64, vp, i64, i64, vp]
    L.ttb_mx_quantize_both.restype = i32
    L.ttb_gemm_mxfp8.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, vp, i32, vp, vp]
    L.ttb_gemm_mxfp8.restype = i32
    L.ttb_fp8_cast_transpose.restype = i32
    for fn in (L.ttb_moe_route_sort, L.ttb_moe_permute_indices, L.ttb_embedding_fwd, L.ttb_embedding_bwd):
        fn.restype = i32
    L.ttb_ensure_device.restype = i32
    L.ttb_launch_count.restype = i64
    L.ttb_attn_bwd.restype = i32
    for fn in (L.ttb_gemm_bf16, L.ttb_rmsnorm_fwd, L.ttb_rmsnorm_bwd, L.ttb_rope, L.ttb_swiglu_fwd, L.ttb_swiglu_bwd, L.ttb_adamw, L.ttb_grad_sumsq, L.ttb_softmax_ce):
        fn.restype = i32


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed: {ERROR_NAMES.get(rc, rc)}")


def stream_ptr() -> int:
    """Handle of torch's current stream.  Also binds the calling thread (autograd workers
    included) to torch's current device inside the kernel library, whose CUDA runtime keeps
    its own per-thread device state."""
    lib().ttb_ensure_device(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def err_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels set when one of their bounded waits gives up."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _err_words:
        _err_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_words[key]


def index_violations(reset: bool = True) -> int:
    """Out-of-range token ids, labels and positions that kernels replaced by a safe value (row 0 / ignored / position 0) since the
    last reset, on the current device.  Synchronises."""
    return int(lib().ttb_index_violations(int(reset)))


def check_device_errors(device: Optional[torch.device] = None) -> None:
    """Synchronising check of the device error word; raises if any kernel timed out.  With ``TTB_DEBUG_BOUNDS=1`` an out-of-range
    user index seen by a kernel raises too."""
    if os.environ.get("TTB_DEBUG_BOUNDS", "0") == "1" and _err_words:
        n = index_violations()
        if n:
            raise KernelError(f"{n} out-of-range token ids / labels / positions were replaced by safe values (TTB_DEBUG_BOUNDS=1)")
    for key, word in _err_words.items():
        code = int(word.item())
        if code != 0:
            word.zero_()
            raise KernelError(f"a kernel on cuda:{key} gave up waiting (site code {code}); results are invalid")

