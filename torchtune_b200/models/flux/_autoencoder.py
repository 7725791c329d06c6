"""Flux.1 image autoencoder (parity: torchtune/models/flux/_autoencoder.py:16-330): a convolutional
VAE — ResNet blocks with GroupNorm/SiLU, strided-conv down-sampling, nearest-neighbour up-sampling, one
single-head attention layer at the lowest resolution — whose latent is shifted and scaled for the
diffusion model.  Module names follow the reference so its converted checkpoints load directly."""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...modules import Linear, MultiHeadAttention


def _norm(ch: int) -> nn.GroupNorm:
    return nn.GroupNorm(num_groups=32, num_channels=ch, eps=1e-6, affine=True)


def _conv3(ch_in: int, ch_out: int, stride: int = 1, padding: int = 1) -> nn.Conv2d:
    return nn.Conv2d(ch_in, ch_out, kernel_size=3, stride=stride, padding=padding)


class ResnetLayer(nn.Module):
    def __init__(self, ch_in: int, ch_out: int):
        super().__init__()
        self.main = nn.Sequential(_norm(ch_in), nn.SiLU(), _conv3(ch_in, ch_out), _norm(ch_out), nn.SiLU(), _conv3(ch_out, ch_out))
        self.shortcut = nn.Identity() if ch_in == ch_out else nn.Conv2d(ch_in, ch_out, kernel_size=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.main(x) + self.shortcut(x)


class AttnLayer(nn.Module):
    """Single-head self-attention over all pixels of the feature map."""

    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim
        self.norm = _norm(dim)
        self.attn = MultiHeadAttention(embed_dim=dim, num_heads=1, num_kv_heads=1, head_dim=dim, q_proj=Linear(dim, dim), k_proj=Linear(dim, dim), v_proj=Linear(dim, dim), output_proj=Linear(dim, dim), is_causal=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, c, h, w = x.shape
        seq = self.norm(x).permute(0, 2, 3, 1).reshape(b, h * w, c)
        out = self.attn(seq, seq).reshape(b, h, w, c).permute(0, 3, 1, 2)
        return out + x


class Downsample(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = _conv3(ch, ch, stride=2, padding=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.conv(F.pad(x, (0, 1, 0, 1)))  # asymmetric padding: right / bottom only


class Upsample(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = _conv3(ch, ch)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


def resnet_layers(n: int, ch_in: int, ch_out: int) -> nn.Sequential:
    return nn.Sequential(*[ResnetLayer(ch_in if i == 0 else ch_out, ch_out) for i in range(n)])


class DownBlock(nn.Module):
    def __init__(self, n_layers: int, ch_in: int, ch_out: int, downsample: bool):
        super().__init__()
        self.layers = resnet_layers(n_layers, ch_in, ch_out)
        self.downsample = Downsample(ch_out) if downsample else nn.Identity()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.downsample(self.layers(x))


class UpBlock(nn.Module):
    def __init__(self, n_layers: int, ch_in: int, ch_out: int, upsample: bool):
        super().__init__()
        self.layers = resnet_layers(n_layers, ch_in, ch_out)
        self.upsample = Upsample(ch_out) if upsample else nn.Identity()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.upsample(self.layers(x))


def mid_block(ch: int) -> nn.Sequential:
    return nn.Sequential(ResnetLayer(ch, ch), AttnLayer(ch), ResnetLayer(ch, ch))


def end_block(ch_in: int, ch_out: int) -> nn.Sequential:
    return nn.Sequential(_norm(ch_in), nn.SiLU(), _conv3(ch_in, ch_out))


def diagonal_gaussian(z: torch.Tensor) -> torch.Tensor:
    """Sample from the Gaussian whose mean / log-variance are the two channel halves of ``z``."""
    mean, logvar = torch.chunk(z, 2, dim=1)
    return mean + torch.exp(0.5 * logvar) * torch.randn_like(mean)


class FluxEncoder(nn.Module):
    def __init__(self, ch_in: int, ch_z: int, channels: List[int], n_layers_per_down_block: int, scale_factor: float, shift_factor: float):
        super().__init__()
        self.scale_factor, self.shift_factor = scale_factor, shift_factor
        self.conv_in = _conv3(ch_in, channels[0])
        self.down = nn.ModuleList(DownBlock(n_layers_per_down_block, channels[max(i - 1, 0)], channels[i], downsample=i < len(channels) - 1) for i in range(len(channels)))
        self.mid = mid_block(channels[-1])
        self.end = end_block(channels[-1], 2 * ch_z)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.conv_in(x)
        for block in self.down:
            h = block(h)
        z = diagonal_gaussian(self.end(self.mid(h)))
        return self.scale_factor * (z - self.shift_factor)


class FluxDecoder(nn.Module):
    def __init__(self, ch_out: int, ch_z: int, channels: List[int], n_layers_per_up_block: int, scale_factor: float, shift_factor: float):
        super().__init__()
        self.scale_factor, self.shift_factor = scale_factor, shift_factor
        self.conv_in = _conv3(ch_z, channels[0])
        self.mid = mid_block(channels[0])
        self.up = nn.ModuleList(UpBlock(n_layers_per_up_block, channels[max(i - 1, 0)], channels[i], upsample=i < len(channels) - 1) for i in range(len(channels)))
        self.end = end_block(channels[-1], ch_out)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        h = self.mid(self.conv_in(z / self.scale_factor + self.shift_factor))
        for block in self.up:
            h = block(h)
        return self.end(h)


class FluxAutoencoder(nn.Module):
    def __init__(self, img_shape: Tuple[int, int, int], encoder: nn.Module, decoder: nn.Module):
        super().__init__()
        self._img_shape = tuple(img_shape)
        self.encoder, self.decoder = encoder, decoder

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        assert tuple(x.shape[1:]) == self._img_shape, f"expected images of shape {self._img_shape}, got {tuple(x.shape[1:])}"
        return self.encoder(x)

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.decode(self.encode(x))
