"""Positional embeddings of the tiled CLIP vision encoder
(parity: torchtune/models/clip/_position_embeddings.py:16-670).

* :class:`TokenPositionalEmbedding` — one vector per patch (+CLS) for untiled images.
* :class:`TiledTokenPositionalEmbedding` — a local per-patch table shared by all tiles, blended
  (``tanh(gate)``) with a global table indexed by the tile's row/column in the image.
* :class:`TilePositionalEmbedding` — one gated vector per tile position.

Checkpoints trained with a different tile grid or tile size are adapted on load by bilinear
interpolation of the tables (``_load_state_dict_hook``), as the reference does.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn.functional as F
from torch import nn


class TokenPositionalEmbedding(nn.Module):
    def __init__(self, embed_dim: int, tile_size: int, patch_size: int) -> None:
        super().__init__()
        grid = tile_size // patch_size
        self.positional_embedding = nn.Parameter(embed_dim**-0.5 * torch.randn(grid * grid + 1, embed_dim))

    def forward(self, x: torch.Tensor, *args: Any) -> torch.Tensor:
        return x + self.positional_embedding.to(x.dtype)


def _interp_grid(table: torch.Tensor, out_hw) -> torch.Tensor:
    """Bilinear resize of ``[H, W, C]`` to ``[h, w, C]`` (align_corners=True), in fp32."""
    t = table.float().permute(2, 0, 1).unsqueeze(0)
    t = F.interpolate(t, size=out_hw, mode="bilinear", align_corners=True)
    return t.squeeze(0).permute(1, 2, 0).to(table.dtype)


class TiledTokenPositionalEmbedding(nn.Module):
    def __init__(self, max_num_tiles: int, embed_dim: int, tile_size: int, patch_size: int) -> None:
        super().__init__()
        grid = tile_size // patch_size
        self.n_tokens_per_tile = grid * grid + 1
        scale = embed_dim**-0.5
        self.local_token_positional_embedding = nn.Parameter(scale * torch.randn(self.n_tokens_per_tile, embed_dim))
        self.global_token_positional_embedding = nn.Parameter(scale * torch.randn(max_num_tiles, max_num_tiles, self.n_tokens_per_tile, embed_dim))
        self.gate = nn.Parameter(torch.zeros(1))
        self._register_load_state_dict_pre_hook(self._load_state_dict_hook)

    # -- checkpoint adaptation ------------------------------------------------------------
    @staticmethod
    def _resize_local(local: torch.Tensor, n_tokens: int) -> torch.Tensor:
        """The CLS row is kept; the patch rows are treated as a square grid and interpolated."""
        cls, patches = local[:1], local[1:]
        src, dst = int(math.sqrt(patches.shape[0])), int(math.sqrt(n_tokens - 1))
        grid = _interp_grid(patches.reshape(src, src, -1), (dst, dst))
        return torch.cat([cls, grid.reshape(dst * dst, -1)], dim=0)

    @staticmethod
    def _resize_global(glob: torch.Tensor, max_tiles: int, n_tokens: int) -> torch.Tensor:
        """``[T, T, tokens, C]``: patches of all tiles form one ``(T·g)×(T·g)`` image that is
        interpolated as a whole; CLS vectors are interpolated over the tile grid."""
        t_src, _, tok_src, c = glob.shape
        g_src, g_dst = int(math.sqrt(tok_src - 1)), int(math.sqrt(n_tokens - 1))
        cls = _interp_grid(glob[:, :, 0, :], (max_tiles, max_tiles)).unsqueeze(2)
        patches = glob[:, :, 1:, :].reshape(t_src, t_src, g_src, g_src, c).permute(0, 2, 1, 3, 4).reshape(t_src * g_src, t_src * g_src, c)
        patches = _interp_grid(patches, (max_tiles * g_dst, max_tiles * g_dst))
        patches = patches.reshape(max_tiles, g_dst, max_tiles, g_dst, c).permute(0, 2, 1, 3, 4).reshape(max_tiles, max_tiles, g_dst * g_dst, c)
        return torch.cat([cls, patches], dim=2)

    def _load_state_dict_hook(self, state_dict, prefix, *args: Any) -> None:
        local = state_dict.get(prefix + "local_token_positional_embedding")
        if local is not None and local.shape != self.local_token_positional_embedding.shape:
            if local.shape[1] != self.local_token_positional_embedding.shape[1]:
                raise ValueError("local_token_positional_embedding: embedding dimension of the checkpoint does not match the model")
            state_dict[prefix + "local_token_positional_embedding"] = self._resize_local(local, self.n_tokens_per_tile)
        glob = state_dict.get(prefix + "global_token_positional_embedding")
        if glob is not None and glob.shape != self.global_token_positional_embedding.shape:
            if glob.shape[-1] != self.global_token_positional_embedding.shape[-1] or glob.shape[0] != glob.shape[1]:
                raise ValueError("global_token_positional_embedding: checkpoint table has an incompatible shape")
            state_dict[prefix + "global_token_positional_embedding"] = self._resize_global(glob, self.global_token_positional_embedding.shape[0], self.n_tokens_per_tile)

    def forward(self, x: torch.Tensor, aspect_ratio: torch.Tensor) -> torch.Tensor:
        """``x``: ``[bsz·n_imgs, n_tiles, tokens, dim]``; ``aspect_ratio``: ``[bsz·n_imgs, 2]`` (tile rows, cols)."""
        gate = self.gate.tanh().to(x.dtype)
        x = x + self.local_token_positional_embedding.to(x.dtype) * (1 - gate)
        out = x.clone()
        for i, (th, tw) in enumerate(aspect_ratio.tolist()):
            th, tw = int(th), int(tw)
            n = th * tw
            pos = self.global_token_positional_embedding[:th, :tw].reshape(n, self.n_tokens_per_tile, -1).to(x.dtype)
            out[i, :n] = out[i, :n] + pos * gate
        return out


class TilePositionalEmbedding(nn.Module):
    def __init__(self, max_num_tiles: int, embed_dim: int):
        super().__init__()
        self.max_num_tiles, self.embed_dim = max_num_tiles, embed_dim
        self.embedding = nn.Parameter(embed_dim**-0.5 * torch.randn(max_num_tiles, max_num_tiles, 1, embed_dim))
        self.gate = nn.Parameter(torch.zeros(1))
        self._register_load_state_dict_pre_hook(self._load_state_dict_hook)

    def _load_state_dict_hook(self, state_dict, prefix, *args: Any) -> None:
        emb = state_dict.get(prefix + "embedding")
        if emb is not None and emb.shape != self.embedding.shape:
            if emb.shape[-1] != self.embed_dim or emb.shape[0] != emb.shape[1]:
                raise ValueError("tile positional embedding of the checkpoint has an incompatible shape")
            state_dict[prefix + "embedding"] = _interp_grid(emb[:, :, 0, :], (self.max_num_tiles, self.max_num_tiles)).unsqueeze(2)

    def forward(self, x: torch.Tensor, aspect_ratio: torch.Tensor) -> torch.Tensor:
        gate = self.gate.tanh().to(x.dtype)
        out = x.clone()
        for i, (th, tw) in enumerate(aspect_ratio.tolist()):
            th, tw = int(th), int(tw)
            n = th * tw
            pos = self.embedding[:th, :tw].reshape(n, 1, self.embed_dim).to(x.dtype)
            out[i, :n] = out[i, :n] + pos * gate
        return out
