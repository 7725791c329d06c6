"""Rotary position embeddings.

Parity: torchtune/modules/position_embeddings.py:13-258 (interleaved-pair RoPE and
the 2-D vision variant), torchtune/models/llama3_1/_position_embeddings.py:15-190
and torchtune/models/llama4/_position_embeddings.py:15-196 (frequency-scaled
variants), torchtune/models/phi3/_position_embeddings.py:14 and
torchtune/models/qwen2/_positional_embeddings.py:14 (half-split layout).

All variants share one cache format, ``[max_seq_len, dim/2, 2]`` fp32 (cos, sin),
consumed by :func:`torchtune_b200.ops.rope`; inputs are ``[b, s, n_heads, head_dim]``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .. import ops


class RotaryPositionalEmbeddings(nn.Module):
    """Interleaved-pair rotation ``(x[2i], x[2i+1])`` by ``pos * base^(-2i/dim)``."""

    interleaved = True

    def __init__(self, dim: int, max_seq_len: int = 4096, base: float = 10_000) -> None:
        super().__init__()
        self.dim = dim
        self.base = base
        self.max_seq_len = max_seq_len
        self.rope_init()

    # frequency hook -----------------------------------------------------
    def _frequencies(self, device) -> torch.Tensor:
        exponent = torch.arange(0, self.dim, 2, device=device)[: self.dim // 2].float() / self.dim
        return 1.0 / (self.base**exponent)

    def rope_init(self) -> None:
        """(Re)build the non-persistent buffers; safe to call after meta-device construction."""
        dev = None
        existing = getattr(self, "theta", None)
        if existing is not None and existing.device.type != "meta":
            dev = existing.device
        theta = self._frequencies(dev)
        self.register_buffer("theta", theta, persistent=False)
        self.build_rope_cache(self.max_seq_len)

    def build_rope_cache(self, max_seq_len: int = 4096) -> None:
        pos = torch.arange(max_seq_len, dtype=self.theta.dtype, device=self.theta.device)
        angles = torch.einsum("i,j->ij", pos, self.theta).float()
        self.register_buffer("cache", torch.stack([angles.cos(), angles.sin()], dim=-1), persistent=False)
        self.is_cache_built = True

    def forward(self, x: torch.Tensor, *, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rope(x, self.cache, input_pos, interleaved=self.interleaved)


class _ScaledRoPE(RotaryPositionalEmbeddings):
    """Wavelength-dependent frequency scaling used by Llama 3.1 and Llama 4: long
    wavelengths are divided by ``scale_factor``, short ones kept, the band in between
    interpolated smoothly."""

    def __init__(
        self,
        dim: int,
        max_seq_len: int,
        base: float,
        scale_factor: float,
        low_freq_factor: float,
        high_freq_factor: float,
        old_context_len: int,
    ) -> None:
        self.scale_factor = scale_factor
        self.low_freq_factor = low_freq_factor
        self.high_freq_factor = high_freq_factor
        self.old_context_len = old_context_len
        self.is_cache_built = False
        super().__init__(dim, max_seq_len, base)

    def _frequencies(self, device) -> torch.Tensor:
        freqs = super()._frequencies(device)
        return self.apply_scaling(
            freqs, self.scale_factor, self.low_freq_factor, self.high_freq_factor, self.old_context_len
        )

    @staticmethod
    def apply_scaling(freqs, scale_factor, low_freq_factor, high_freq_factor, old_context_len) -> torch.Tensor:
        wavelen = 2 * math.pi / freqs
        low_wl = old_context_len / low_freq_factor
        high_wl = old_context_len / high_freq_factor
        if high_freq_factor == low_freq_factor:
            smooth = torch.zeros_like(freqs)
        else:
            smooth = (old_context_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
        mid = (1 - smooth) * freqs / scale_factor + smooth * freqs
        out = torch.where(wavelen < high_wl, freqs, torch.where(wavelen > low_wl, freqs / scale_factor, mid))
        return out.to(freqs.dtype)


class Llama3ScaledRoPE(_ScaledRoPE):
    def __init__(
        self,
        dim: int,
        max_seq_len: int = 4096,
        base: float = 10_000,
        scale_factor: float = 8,
        low_freq_factor: float = 1,
        high_freq_factor: float = 4,
        old_context_len: int = 8192,
    ) -> None:
        super().__init__(dim, max_seq_len, base, scale_factor, low_freq_factor, high_freq_factor, old_context_len)


class Llama4ScaledRoPE(_ScaledRoPE):
    def __init__(
        self,
        dim: int,
        max_seq_len: int = 4096,
        base: float = 10_000,
        scale_factor: float = 16,
        low_freq_factor: float = 1,
        high_freq_factor: float = 1,
        old_context_len: int = 8192,
    ) -> None:
        super().__init__(dim, max_seq_len, base, scale_factor, low_freq_factor, high_freq_factor, old_context_len)


class HalfSplitRotaryPositionalEmbeddings(RotaryPositionalEmbeddings):
    """Rotation of pairs ``(x[i], x[i + dim/2])`` — the layout HF checkpoints of Qwen and
    Phi use, so no q/k permutation is needed when loading them."""

    interleaved = False


class Qwen2RotaryPositionalEmbeddings(HalfSplitRotaryPositionalEmbeddings):
    def __init__(self, dim: int, max_seq_len: int = 4096, base: float = 1_000_000.0) -> None:
        super().__init__(dim, max_seq_len, base)


class Phi3RotaryPositionalEmbeddings(HalfSplitRotaryPositionalEmbeddings):
    def __init__(self, dim: int, max_seq_len: int = 4096, base: float = 10_000) -> None:
        super().__init__(dim, max_seq_len, base)


class VisionRotaryPositionalEmbeddings(nn.Module):
    """2-D RoPE over a ``patch_grid x patch_grid`` image: the first half of the head
    dimension rotates with the patch's x index, the second half with its y index; the
    CLS slot (last position of every tile) is left unrotated."""

    def __init__(
        self, patch_size: int, tile_size: int, max_num_tiles: int, dim: int, base: float = 10_000, append_cls_token: bool = True
    ) -> None:
        super().__init__()
        self.patch_grid_size = tile_size // patch_size
        self.max_num_tiles = max_num_tiles
        self.dim = dim
        self.base = base
        self.append_cls_token = append_cls_token
        self.rope_init()

    def rope_init(self) -> None:
        exponent = torch.arange(0, self.dim, 2)[: self.dim // 2].float() / self.dim
        self.register_buffer("theta", 1.0 / (self.base**exponent), persistent=False)
        self.build_rope_cache()

    def build_rope_cache(self) -> None:
        g = self.patch_grid_size
        n = g * g
        idx = torch.arange(n + 1, dtype=self.theta.dtype, device=self.theta.device)
        idx = torch.cat([idx[-1:], idx[:-1]]) if not self.append_cls_token else idx
        is_cls = idx == n
        px = (idx % g).masked_fill(is_cls, -1)
        py = (idx // g).masked_fill(is_cls, -1)
        # each axis uses every other frequency so x and y together fill dim/2 slots
        fx = torch.einsum("i,j->ij", px + 1, self.theta[0::2]).float()
        fy = torch.einsum("i,j->ij", py + 1, self.theta[0::2]).float()
        ang = torch.cat([fx, fy], dim=-1)
        ang = ang.masked_fill(is_cls.unsqueeze(-1), 0.0)
        self.register_buffer("cache", torch.stack([ang.cos(), ang.sin()], dim=-1), persistent=False)

    def forward(self, x: torch.Tensor, **kwargs) -> torch.Tensor:
        """``x``: ``[b, s, n_heads, head_dim]`` where ``s = n_tiles * (grid^2 + 1)``."""
        b, s, h, d = x.shape
        per_tile = self.cache.shape[0]
        pos = torch.arange(s, device=x.device) % per_tile
        return ops.rope(x, self.cache, pos.unsqueeze(0).expand(b, s), interleaved=True)
