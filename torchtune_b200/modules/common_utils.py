"""KV-cache context managers and state-dict helpers (parity: torchtune/modules/common_utils.py:24-444)."""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Generator, List, Optional

import torch
from torch import nn


def reparametrize_as_dtype_state_dict_post_hook(
    model: nn.Module, state_dict: Dict[str, Any], *args: Any, dtype: torch.dtype = torch.bfloat16, offload_to_cpu: bool = True, **kwargs: Any
) -> None:
    """State-dict post hook that stores every floating tensor in ``dtype`` (optionally on
    CPU).  NF4 layers of this package already expose dense weights in their state dict,
    so this only normalises dtype/device."""
    for k, v in list(state_dict.items()):
        if isinstance(v, torch.Tensor) and v.is_floating_point():
            v = v.to(dtype)
            state_dict[k] = v.cpu() if offload_to_cpu else v


def _register_reparametrize_state_dict_hooks(module: nn.Module, dtype: torch.dtype = torch.bfloat16, offload_to_cpu: bool = True) -> None:
    import functools

    module._register_state_dict_hook(
        functools.partial(reparametrize_as_dtype_state_dict_post_hook, dtype=dtype, offload_to_cpu=offload_to_cpu)
    )


def slice_str_to_array(slice_str: str, length: int) -> List[bool]:
    """``"1:3"``, ``"::2"``, ``"0,4,5"`` … → boolean membership list of ``length``."""
    assert "," not in slice_str or ":" not in slice_str, "Cannot mix commas and colons"
    flags = [False] * length
    if "," in slice_str:
        picks = [int(tok) for tok in slice_str.split(",")]
        assert all(0 <= i < length for i in picks), "Index out of range"
        for i in picks:
            flags[i] = True
        return flags
    fields = slice_str.split(":")
    assert len(fields) <= 3, "Invalid slice format"
    nums: List[Optional[int]] = [int(f) if f != "" else None for f in fields]
    if len(fields) == 1:
        start = nums[0]
        stop, step = (None, None) if start is None else (start + 1, 1)
    else:
        start, stop = nums[0], nums[1]
        step = nums[2] if len(fields) == 3 else None
    assert start is None or 0 <= start < length, "Start index out of range"
    assert stop is None or 0 <= stop < length or (len(fields) == 1), "End index out of range"
    assert step is None or step != 0, "Step cannot be zero"
    for i in range(0 if start is None else start, length if stop is None else stop, 1 if step is None else step):
        if 0 <= i < length:
            flags[i] = True
    return flags


def _attention_modules(model: nn.Module):
    from .attention import MultiHeadAttention

    return [m for m in model.modules() if isinstance(m, MultiHeadAttention)]


@contextlib.contextmanager
def disable_kv_cache(model: nn.Module) -> Generator[None, None, None]:
    """Temporarily run a cache-equipped model as if it had no KV caches (the buffers are
    kept and re-enabled on exit)."""
    if not model.caches_are_setup():
        raise ValueError("Model caches must be setup before calling disable_kv_cache! Please use model.setup_caches()")
    if not model.caches_are_enabled():
        import warnings

        warnings.warn("You are using disable_kv_cache with a model that does not have caches enabled. This is a no-op and the expected behaviour may not occur.")
    mods = _attention_modules(model)
    for m in mods:
        m.cache_enabled = False
    try:
        yield
    finally:
        for m in mods:
            if m.kv_cache is not None:
                m.cache_enabled = True


@contextlib.contextmanager
def local_kv_cache(
    model: nn.Module,
    *,
    batch_size: int,
    device: torch.device,
    dtype: torch.dtype,
    encoder_max_seq_len: Optional[int] = None,
    decoder_max_seq_len: Optional[int] = None,
) -> Generator[None, None, None]:
    """Create KV caches for the duration of the block and delete them afterwards."""
    if model.caches_are_setup():
        raise ValueError("Model caches must be not setup prior to entering this context manager! Please use delete_kv_caches(model) to delete existing caches.")
    with device:
        model.setup_caches(batch_size, dtype, encoder_max_seq_len=encoder_max_seq_len, decoder_max_seq_len=decoder_max_seq_len)
    try:
        yield
    finally:
        delete_kv_caches(model)


def delete_kv_caches(model: nn.Module) -> None:
    if not model.caches_are_setup():
        raise ValueError("You have tried to delete model caches, but model.caches_are_setup() is False! Please setup caches on the model first.")
    for m in _attention_modules(model):
        if m.kv_cache is not None:
            m.cache_enabled = False
            m.kv_cache = None
