"""Qwen3 attention as a class of its own (parity: torchtune/models/qwen3/_attention.py:17-250).

The only difference from the shared attention module is the order of two steps: q and k are normalised per head *before* the rotary
embedding.  The shared module has that as a switch (the whole-model builders set it); this class fixes it on, for callers who build
layers by hand under the reference's name."""
from ...modules.attention import MultiHeadAttention


class Qwen3Attention(MultiHeadAttention):
    def __init__(self, **kwargs) -> None:
        kwargs.setdefault("qk_norm_before_rope", True)
        super().__init__(**kwargs)
