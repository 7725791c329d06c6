"""Tiled vision transformer (parity: torchtune/modules/vision_transformer.py:16-470).

Input images are pre-cut into tiles; every tile is split into ``patch_grid²`` patches, a CLS
slot is added per tile, and all tiles of an image attend to each other in one sequence.
State-dict keys match the reference (``conv.weight``, ``ln_pre``, ``ln_post``,
``cls_token_embedding.weight``, ``layers.N…``).

The patch embedding — a convolution whose stride equals its kernel — is evaluated as what it
is, a matrix product ``[tiles·patches, C·p·p] × [C·p·p, embed]``, so on bf16 CUDA tensors it
runs on the same tcgen05 GEMM as every other projection.
"""
from __future__ import annotations

import copy
from typing import List, Optional, Tuple

import torch
from torch import nn

from .. import ops
from .layer_norm import Fp32LayerNorm


class PatchEmbedding(nn.Module):
    """``nn.Conv2d(in_channels, embed_dim, kernel=stride=patch)`` expressed as unfold + GEMM; the
    parameter keeps the convolution's name and shape (``weight [embed, C, p, p]``)."""

    def __init__(self, in_channels: int, embed_dim: int, patch_size: int, bias: bool = False):
        super().__init__()
        self.in_channels, self.embed_dim, self.patch_size = in_channels, embed_dim, patch_size
        ref = nn.Conv2d(in_channels, embed_dim, kernel_size=(patch_size, patch_size), stride=(patch_size, patch_size), bias=bias)
        self.weight = ref.weight
        self.bias = ref.bias

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """``[n, C, H, W]`` → ``[n, (H/p)·(W/p), embed]``."""
        n, c, h, w = images.shape
        p = self.patch_size
        gh, gw = h // p, w // p
        patches = images[:, :, : gh * p, : gw * p].reshape(n, c, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(n * gh * gw, c * p * p)
        k = patches.shape[1]
        wmat = self.weight.reshape(self.embed_dim, k)
        pad = (-k) % 8
        if pad and patches.is_cuda:  # GEMM rows must be 16-byte multiples
            patches = torch.nn.functional.pad(patches, (0, pad))
            wmat = torch.nn.functional.pad(wmat, (0, pad))
        out = ops.linear(patches.contiguous(), wmat.contiguous(), self.bias)
        return out.reshape(n, gh * gw, self.embed_dim)


class CLSEmbedding(nn.Module):
    """One learned vector added as an extra token to every tile (front, or back when
    ``append_cls_token``)."""

    def __init__(self, embed_dim: int, append_cls_token: bool = False) -> None:
        super().__init__()
        self.weight = nn.Parameter(embed_dim**-0.5 * torch.randn(embed_dim))
        self.append_cls_token = append_cls_token

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n, tiles, _, dim = x.shape
        cls = self.weight.to(x.dtype).expand(n, tiles, 1, dim)
        return torch.cat([x, cls], dim=2) if self.append_cls_token else torch.cat([cls, x], dim=2)


class CLSProjection(nn.Module):
    """Keeps only the (front) CLS token of every tile and projects it to ``cls_output_dim``."""

    def __init__(self, embed_dim: int, cls_output_dim: int) -> None:
        super().__init__()
        self.cls_output_dim = cls_output_dim
        self.weight = nn.Parameter(embed_dim**-0.5 * torch.randn(embed_dim, cls_output_dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bsz, n_imgs, n_tiles, _, dim = x.shape
        cls = x[:, :, :, 0, :].reshape(bsz * n_imgs * n_tiles, dim)
        return (cls @ self.weight.to(cls.dtype)).reshape(bsz, n_imgs, n_tiles, 1, self.cls_output_dim)


class VisionTransformer(nn.Module):
    def __init__(
        self,
        patch_size: int,
        tile_size: int,
        num_layers: int,
        embed_dim: int,
        layer: nn.Module,
        token_pos_embedding: nn.Module,
        pre_tile_pos_embed: Optional[nn.Module] = None,
        post_tile_pos_embed: Optional[nn.Module] = None,
        cls_projection: Optional[nn.Module] = None,
        out_indices: Optional[List[int]] = None,
        in_channels: int = 3,
        append_cls_token: bool = False,
    ) -> None:
        super().__init__()
        if tile_size <= 0:
            raise ValueError("tile_size must be > 0")
        if patch_size <= 0:
            raise ValueError("patch_size must be > 0")
        if out_indices and len(out_indices) > num_layers:
            raise ValueError(f"len(out_indices) must be <= num_layers. Got out_indices={out_indices!r} and num_layers={num_layers!r}")
        grid = tile_size // patch_size
        self.patches_per_tile = grid * grid
        self.out_indices = list(out_indices) if out_indices else []
        self.pre_tile_pos_embed = pre_tile_pos_embed
        self.post_tile_pos_embed = post_tile_pos_embed
        self.token_pos_embedding = token_pos_embedding
        self.cls_projection = cls_projection
        self.layers = nn.ModuleList([copy.deepcopy(layer) for _ in range(num_layers)])
        self.conv = PatchEmbedding(in_channels, embed_dim, patch_size, bias=False)
        self.ln_post = Fp32LayerNorm(embed_dim)
        self.ln_pre = Fp32LayerNorm(embed_dim)
        self.cls_token_embedding = CLSEmbedding(embed_dim, append_cls_token=append_cls_token)

    def get_image_tokens_per_tile(self) -> int:
        return self.patches_per_tile + 1

    def forward(self, images: torch.Tensor, aspect_ratio: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """``images``: ``[bsz, n_imgs, n_tiles, C, H, W]``; ``aspect_ratio``: ``[bsz, n_imgs, 2]`` tile grid of
        every image (``None`` when images are not tiled).  Returns ``(tokens [bsz, n_imgs, n_tiles,
        n_tokens, dim], hidden_states)`` with one hidden state per entry of ``out_indices`` (the input
        of that layer; index ``num_layers`` = output of the last layer)."""
        bsz, n_imgs, n_tiles, nch, height, width = images.shape
        n = bsz * n_imgs
        if aspect_ratio is not None:
            aspect_ratio = aspect_ratio.reshape(n, 2)
        x = self.conv(images.reshape(n * n_tiles, nch, height, width)).reshape(n, n_tiles, self.patches_per_tile, -1)
        dim = x.shape[-1]
        if self.pre_tile_pos_embed is not None:
            x = self.pre_tile_pos_embed(x, aspect_ratio)
        x = self.cls_token_embedding(x)
        n_tokens = x.shape[2]
        x = self.token_pos_embedding(x, aspect_ratio)
        x = self.ln_pre(x)
        x = x.reshape(n, n_tiles * n_tokens, dim)
        hidden: List[torch.Tensor] = []
        for idx, layer in enumerate(self.layers):
            if idx in self.out_indices:
                hidden.append(x.reshape(bsz, n_imgs, n_tiles, n_tokens, dim))
            x = layer(x)
        if len(self.layers) in self.out_indices:
            hidden.append(x.reshape(bsz, n_imgs, n_tiles, n_tokens, dim))
        x = self.ln_post(x)
        if self.post_tile_pos_embed is not None:
            x = self.post_tile_pos_embed(x.reshape(n, n_tiles, n_tokens, dim), aspect_ratio)
        x = x.reshape(bsz, n_imgs, n_tiles, n_tokens, dim)
        if self.cls_projection is not None:
            x = self.cls_projection(x)
        return x, hidden
