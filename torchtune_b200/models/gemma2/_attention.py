"""Gemma-2 attention as a class of its own (parity: torchtune/models/gemma2/_attention.py:17-290).

Three differences from the shared attention module, each of which the shared module or the layer already expresses as data — score
soft-capping ``cap·tanh(s/cap)``, a query scale of ``query_pre_attn_scalar**-0.5`` instead of ``head_dim**-0.5``, and a sliding
window on alternating layers.  The whole-model builder passes the first two as arguments and hangs the window on the layer's mask
hook; this class takes the reference's constructor arguments and applies the window itself, for callers who build layers by hand."""
from typing import Optional

import torch

from ...modules.attention import MultiHeadAttention
from .._factory import _window_mask_mod


class Gemma2Attention(MultiHeadAttention):
    def __init__(self, *, sliding_window_size: Optional[int] = None, softcapping: Optional[float] = 50.0,
                 query_pre_attn_scalar: Optional[int] = None, **kwargs) -> None:
        head_dim = kwargs["head_dim"]
        super().__init__(softcap=float(softcapping or 0.0), scale=float(query_pre_attn_scalar or head_dim) ** -0.5, **kwargs)
        self.sliding_window_size = sliding_window_size
        self.softcapping = softcapping
        self.query_pre_attn_scalar = query_pre_attn_scalar
        self._window = _window_mask_mod(int(sliding_window_size)) if sliding_window_size else None

    def forward(self, x: torch.Tensor, y: Optional[torch.Tensor] = None, *, mask=None, **kwargs) -> torch.Tensor:
        if self._window is not None:
            mask = self._window(mask, x.shape[0], x.shape[1])
        return super().forward(x, y, mask=mask, **kwargs)
