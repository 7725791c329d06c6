"""Llama-4 vision encoder: ViT with 2-D RoPE per tile, pixel-shuffle down-sampling and an MLP
projector (parity: torchtune/models/llama4/_encoder.py:14-130)."""
from __future__ import annotations

import torch
from torch import nn

from ...modules.model_fusion import register_fusion_module


class Llama4VisionProjectionHead(nn.Module):
    """Drops the CLS slot, folds every 2×2 patch neighbourhood into channels (pixel shuffle with
    factor ½: 4× fewer tokens, 4× wider) and projects to the decoder width."""

    def __init__(self, output: nn.Module, pixel_shuffle_scaling_factor: float = 0.5) -> None:
        super().__init__()
        self.output = output
        self.pixel_shuffle_scaling_factor = pixel_shuffle_scaling_factor

    def _pixel_shuffle(self, x: torch.Tensor) -> torch.Tensor:
        f = self.pixel_shuffle_scaling_factor
        n, w, h, c = x.shape
        x = x.reshape(n, w, int(h * f), int(c / f)).permute(0, 2, 1, 3)
        x = x.reshape(n, int(h * f), int(w * f), int(c / (f * f))).permute(0, 2, 1, 3)
        return x.contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x[:, :-1, :]  # CLS is appended last
        bsz, n_patches, _ = x.shape
        side = int(n_patches**0.5)
        x = self._pixel_shuffle(x.reshape(bsz, side, side, -1))
        return self.output(x.reshape(bsz, -1, x.shape[-1]))


class Llama4VisionEncoder(nn.Module):
    """``images [n_tiles_total, C, H, W]`` (every tile is its own "image") → ``[n_tiles_total,
    tokens_per_tile, decoder_dim]``."""

    def __init__(self, clip: nn.Module, projection_head: nn.Module) -> None:
        super().__init__()
        self.clip, self.projection = clip, projection_head
        register_fusion_module(self.projection)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        x, _ = self.clip(images[:, None, None])
        return self.projection(x.squeeze(2).squeeze(1))
