"""Vision encoder of Llama 3.2 Vision: tiled CLIP trunk + projection head
(parity: torchtune/models/llama3_2_vision/_encoder.py:15-130)."""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from ...modules.model_fusion import register_fusion_module


class Llama3VisionProjectionHead(nn.Module):
    """A few more transformer layers over all tokens of an image, then a linear map of the final
    state concatenated with ``num_hidden_inputs`` intermediate CLIP states to the decoder width."""

    def __init__(self, layers: List[nn.Module], output: nn.Module, num_hidden_inputs: int = 0) -> None:
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.output = output
        self.num_hidden = num_hidden_inputs

    def forward(self, x: torch.Tensor, hidden_states: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        bsz, imgs, tiles, embeds, dim = x.shape
        x = x.reshape(bsz * imgs, tiles * embeds, dim)
        for layer in self.layers:
            x = layer(x)
        x = x.reshape(bsz, imgs, tiles, embeds, dim)
        if self.num_hidden > 0:
            extra = torch.stack(hidden_states, dim=-1).reshape(bsz, imgs, tiles, embeds, -1)
            x = torch.cat([x, extra], dim=-1)
        return self.output(x).reshape(bsz, imgs * tiles * embeds, -1)


class Llama3VisionEncoder(nn.Module):
    """``images [b, n_imgs, n_tiles, C, H, W]`` (+ ``aspect_ratio [b, n_imgs, 2]``) →
    ``[b, n_imgs·n_tiles·tokens, decoder_dim]``."""

    def __init__(self, clip: nn.Module, projection_head: nn.Module) -> None:
        super().__init__()
        self.clip, self.projection = clip, projection_head
        register_fusion_module(self.projection)  # the head did not exist in the pre-trained trunk

    def forward(self, images: torch.Tensor, aspect_ratio: Optional[torch.Tensor] = None) -> torch.Tensor:
        x, hidden = self.clip(images, aspect_ratio)
        return self.projection(x, hidden)
