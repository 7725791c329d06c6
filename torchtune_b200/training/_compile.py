"""``compile_model`` / ``compile_loss`` (API parity with torchtune/training/_compile.py:24-75).

The reference speeds models up with a tracing compiler that fuses the eager op chains of each layer.  This package's layers already
run hand-written fused sm_100a kernels (GEMM epilogues, flash attention, fused norm / RoPE / SwiGLU, fused linear + cross-entropy),
so there is nothing for a tracing compiler to fuse on the hot path, and routing the custom kernels through one would only add guards
and graph breaks.  Both functions therefore leave CUDA bf16 models as they are (the ``compile`` recipe flag is accepted and logged).
For models that run on the generic PyTorch path (CPU, fp32) they fall back to ``torch.compile`` when ``TORCHTUNE_B200_COMPILE=1``.
"""
from __future__ import annotations

import os
from typing import Any

import torch
from torch import nn

from ..utils import get_logger

log = get_logger("INFO")


def _generic_path(module: nn.Module) -> bool:
    p = next(module.parameters(), None)
    return p is None or not p.is_cuda or p.dtype != torch.bfloat16


def compile_model(model: nn.Module, verbose: bool = True) -> None:
    core = getattr(model, "decoder", model)
    if _generic_path(core) and os.environ.get("TORCHTUNE_B200_COMPILE") == "1":
        from ..modules import TransformerCrossAttentionLayer, TransformerSelfAttentionLayer

        backend = os.environ.get("TORCH_COMPILE_BACKEND", "inductor")
        if verbose:
            log.info("Compiling model layers with torch.compile. Expect a relatively slower first step.")
        for m in reversed(list(core.modules())):
            if isinstance(m, (TransformerSelfAttentionLayer, TransformerCrossAttentionLayer)):
                m.compile(backend=backend)
    elif verbose:
        log.info("compile=True: layers already run fused sm_100a kernels; no tracing compiler is applied.")


def compile_loss(loss: nn.Module, verbose: bool = True) -> Any:
    if hasattr(loss, "apply_compile_strategy") and os.environ.get("TORCHTUNE_B200_COMPILE") == "1":
        return loss.apply_compile_strategy(backend=os.environ.get("TORCH_COMPILE_BACKEND", "inductor"))
    if verbose:
        log.info("compile=True: the loss already runs the fused linear + cross-entropy kernel; left as is.")
    return loss
