"""Exportable tile / tiled-token positional embeddings (parity: torchtune/modules/_export/_position_embeddings.py:21-740).

The training versions loop over the batch with Python integers read from ``aspect_ratio``; here the per-sample selection is a mask
built with tensor ops (``row < h`` and ``col < w`` over the fixed tile grid), so the graph has no data-dependent control flow."""
from __future__ import annotations

import torch
from torch import nn

from ...models.clip._position_embeddings import TiledTokenPositionalEmbedding as _TrainTiledToken
from ...models.clip._position_embeddings import TilePositionalEmbedding as _TrainTile


def _grid_mask(aspect_ratio: torch.Tensor, max_tiles: int, n_tiles: int) -> torch.Tensor:
    """``[n, n_tiles, max_tiles, max_tiles]`` one-hot: tile ``t`` of sample ``i`` sits at grid cell ``(t // w_i, t % w_i)`` when ``t < h_i·w_i``."""
    h, w = aspect_ratio[:, 0:1], aspect_ratio[:, 1:2].clamp_min(1)
    t = torch.arange(n_tiles, device=aspect_ratio.device).unsqueeze(0)
    row, col = t // w, t % w
    valid = t < h * w
    rows = torch.arange(max_tiles, device=aspect_ratio.device).view(1, 1, -1, 1)
    cols = torch.arange(max_tiles, device=aspect_ratio.device).view(1, 1, 1, -1)
    return ((rows == row[..., None, None]) & (cols == col[..., None, None]) & valid[..., None, None]).to(torch.float32)


class TilePositionalEmbedding(nn.Module):
    def __init__(self, max_num_tiles: int, embed_dim: int):
        super().__init__()
        self.max_num_tiles, self.embed_dim = max_num_tiles, embed_dim
        self.embedding = nn.Parameter(embed_dim**-0.5 * torch.randn(max_num_tiles, max_num_tiles, 1, embed_dim))
        self.gate = nn.Parameter(torch.zeros(1))

    def forward(self, x: torch.Tensor, aspect_ratio: torch.Tensor) -> torch.Tensor:
        n, n_tiles, _, dim = x.shape
        sel = _grid_mask(aspect_ratio, self.max_num_tiles, n_tiles)  # [n, tiles, T, T]
        pos = torch.einsum("ntrc,rcd->ntd", sel, self.embedding[:, :, 0, :].float()).to(x.dtype)
        return x + pos.unsqueeze(2) * self.gate.tanh().to(x.dtype)


class TiledTokenPositionalEmbedding(nn.Module):
    def __init__(self, max_num_tiles: int, embed_dim: int, tile_size: int, patch_size: int) -> None:
        super().__init__()
        self.n_tokens_per_tile = (tile_size // patch_size) ** 2 + 1
        self.max_num_tiles = max_num_tiles
        scale = embed_dim**-0.5
        self.local_token_positional_embedding = nn.Parameter(scale * torch.randn(self.n_tokens_per_tile, embed_dim))
        self.global_token_positional_embedding = nn.Parameter(scale * torch.randn(max_num_tiles, max_num_tiles, self.n_tokens_per_tile, embed_dim))
        self.gate = nn.Parameter(torch.zeros(1))

    def forward(self, x: torch.Tensor, aspect_ratio: torch.Tensor) -> torch.Tensor:
        n, n_tiles, _, dim = x.shape
        gate = self.gate.tanh().to(x.dtype)
        x = x + self.local_token_positional_embedding.to(x.dtype) * (1 - gate)
        sel = _grid_mask(aspect_ratio, self.max_num_tiles, n_tiles)
        pos = torch.einsum("ntrc,rckd->ntkd", sel, self.global_token_positional_embedding.float()).to(x.dtype)
        return x + pos * gate


def _swap(model: nn.Module, src_cls, make) -> nn.Module:
    for name, child in list(model.named_children()):
        if isinstance(child, src_cls):
            new = make(child)
            new.load_state_dict(child.state_dict())
            setattr(model, name, new)
        else:
            _swap(child, src_cls, make)
    return model


def replace_tile_positional_embedding(model: nn.Module) -> nn.Module:
    return _swap(model, _TrainTile, lambda m: TilePositionalEmbedding(m.max_num_tiles, m.embed_dim))


def replace_tiled_token_positional_embedding(model: nn.Module) -> nn.Module:
    def make(m):
        t, _, tokens, dim = m.global_token_positional_embedding.shape
        new = TiledTokenPositionalEmbedding.__new__(TiledTokenPositionalEmbedding)
        nn.Module.__init__(new)
        new.n_tokens_per_tile, new.max_num_tiles = tokens, t
        new.local_token_positional_embedding = nn.Parameter(torch.empty(tokens, dim))
        new.global_token_positional_embedding = nn.Parameter(torch.empty(t, t, tokens, dim))
        new.gate = nn.Parameter(torch.zeros(1))
        return new

    return _swap(model, _TrainTiledToken, make)
