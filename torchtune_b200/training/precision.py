"""dtype selection and default-dtype scoping (parity: torchtune/training/precision.py:18-176)."""
from __future__ import annotations

import contextlib
from typing import Dict, Generator, Iterable, Optional, Tuple

import torch

from ..utils import get_logger

log = get_logger()

PRECISION_STR_TO_DTYPE: Dict[str, torch.dtype] = {
    "fp16": torch.float16,
    "bf16": torch.bfloat16,
    "fp32": torch.float32,
    "fp64": torch.float64,
}


def _set_float32_precision(precision: str = "high") -> None:
    """Allow TF32 for fp32 matmuls/convolutions on CUDA (``highest`` disables it)."""
    if not torch.cuda.is_available():
        return
    torch.set_float32_matmul_precision(precision)
    torch.backends.cudnn.allow_tf32 = precision != "highest"


def verify_bf16_support() -> bool:
    if torch.cuda.is_available():
        return torch.cuda.is_bf16_supported()
    return True  # CPU bf16 emulation is always available in torch


def get_dtype(dtype: Optional[str] = None, device: Optional[torch.device] = None) -> torch.dtype:
    """Map ``"bf16"``/``"fp32"``/… to a ``torch.dtype`` (default fp32), checking bf16 support."""
    if dtype is None:
        return torch.float32
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype not in PRECISION_STR_TO_DTYPE:
        raise ValueError(f"Dtype {dtype} must be one of {', '.join(PRECISION_STR_TO_DTYPE)} for finetuning.")
    out = PRECISION_STR_TO_DTYPE[dtype]
    if out == torch.bfloat16 and device is not None and device.type == "cuda" and not verify_bf16_support():
        raise RuntimeError("bf16 precision was requested but not available on this hardware. Please use fp32 precision instead.")
    return out


@contextlib.contextmanager
def set_default_dtype(dtype: torch.dtype) -> Generator[None, None, None]:
    """Scope ``torch.set_default_dtype`` to a ``with`` block."""
    previous = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        yield
    finally:
        torch.set_default_dtype(previous)


def validate_expected_param_dtype(named_params: Iterable[Tuple[str, torch.nn.Parameter]], dtype: torch.dtype) -> None:
    for name, p in named_params:
        if p.dtype != dtype:
            raise ValueError(f"Parameter {name} has dtype {p.dtype}, but expected {dtype}")
