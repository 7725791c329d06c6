"""Canvas selection and aspect-preserving resize for tiled image models
(parity: torchtune/modules/transforms/vision_utils/{get_canvas_best_fit,get_inscribed_size,
resize_with_pad,pad_dim_to_size,tile_crop}.py).

All functions work on ``[..., C, H, W]`` tensors and use ``torch.nn.functional`` only, so they run
on the device the image lives on.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


def _divisor_pairs(n: int) -> List[Tuple[int, int]]:
    return [(d, n // d) for d in range(1, n + 1) if n % d == 0]


def find_supported_resolutions(max_num_tiles: int, tile_size: int) -> List[Tuple[int, int]]:
    """Every ``(rows·tile, cols·tile)`` canvas with ``rows·cols <= max_num_tiles``; canvases of
    the same aspect ratio are listed together, larger tile counts first."""
    by_ratio: dict = {}
    for tiles in range(max_num_tiles, 0, -1):
        for rows, cols in _divisor_pairs(tiles):
            by_ratio.setdefault(rows / cols, []).append((rows, cols))
    return [(r * tile_size, c * tile_size) for group in by_ratio.values() for r, c in group]


def get_canvas_best_fit(image: torch.Tensor, possible_resolutions: torch.Tensor, resize_to_max_canvas: bool) -> Tuple[int, int]:
    """The canvas the image fits best without distortion: the smallest up-scaling (or the largest,
    with ``resize_to_max_canvas``) if any canvas allows up-scaling, else the mildest down-scaling;
    ties go to the canvas of least area."""
    h, w = image.shape[-2:]
    res = torch.as_tensor(possible_resolutions)
    scales = torch.minimum(res[:, 0] / h, res[:, 1] / w)
    up = scales[scales >= 1]
    if up.numel():
        chosen = up.max() if resize_to_max_canvas else up.min()
    else:
        chosen = scales[scales < 1].max()
    cands = res[scales == chosen]
    best = cands[(cands[:, 0] * cands[:, 1]).argmin()]
    return int(best[0]), int(best[1])


def get_inscribed_size(image_size: Sequence[int], target_size: Sequence[int], max_size: Optional[int]) -> Tuple[int, int]:
    """Largest size with the image's aspect ratio that fits ``target_size``; ``max_size`` caps how
    far a small image may be up-scaled."""
    assert len(image_size) == 2, "Image size must be a list of length 2."
    assert len(target_size) == 2, "Canvas size must be a list of length 2."
    ih, iw = image_size
    th, tw = target_size
    if max_size is not None:
        th, tw = min(max(ih, max_size), th), min(max(iw, max_size), tw)
    return min(math.floor(ih * (tw / iw)), th), min(math.floor(iw * (th / ih)), tw)


def _fit_without_distortion(image_size: Tuple[int, int], target_size: Tuple[int, int]) -> Tuple[int, int]:
    ih, iw = image_size
    th, tw = target_size
    sw, sh = tw / iw, th / ih
    if sw < sh:
        return min(math.floor(ih * sw), th), tw
    return th, min(math.floor(iw * sh), tw)


_MODES = {"nearest": "nearest", "nearest_exact": "nearest-exact", "bilinear": "bilinear", "bicubic": "bicubic"}


def resize(image: torch.Tensor, size: Tuple[int, int], resample: str = "bilinear") -> torch.Tensor:
    """Antialiased resize of ``[..., C, H, W]`` (float result for float input; uint8 is rounded back)."""
    mode = _MODES[str(resample).lower().split(".")[-1]]
    lead = image.shape[:-3]
    x = image.reshape(-1, *image.shape[-3:])
    was_int = not x.is_floating_point()
    x = x.float() if was_int else x
    kw = dict(antialias=True, align_corners=False) if mode in ("bilinear", "bicubic") else {}
    y = F.interpolate(x, size=tuple(size), mode=mode, **kw)
    if was_int:
        y = y.round().clamp(0, 255).to(image.dtype)
    return y.reshape(*lead, *y.shape[-3:])


def resize_with_pad(image: torch.Tensor, target_size: Tuple[int, int], resample: str = "bilinear", max_size: Optional[int] = None) -> torch.Tensor:
    """Resize preserving the aspect ratio, then zero-pad at the bottom / right to ``target_size``."""
    ih, iw = image.shape[-2:]
    limit = (min(max(ih, max_size), target_size[0]), min(max(iw, max_size), target_size[1])) if max_size is not None else tuple(target_size)
    image = resize(image, _fit_without_distortion((ih, iw), limit), resample)
    h, w = image.shape[-2:]
    return F.pad(image, (0, target_size[1] - w, 0, target_size[0] - h))


def pad_dim_to_size(x: torch.Tensor, size: int, dim: int, fill: float = 0.0) -> torch.Tensor:
    """Right-pad dimension ``dim`` with ``fill`` up to ``size``."""
    cur = x.shape[dim]
    if cur > size:
        raise ValueError(f"dimension {dim} has size {cur}, larger than the requested {size}")
    if cur == size:
        return x
    dim = dim % x.dim()
    pad = [0, 0] * (x.dim() - dim - 1) + [0, size - cur]
    return F.pad(x, pad, value=fill)


def tile_crop(image: torch.Tensor, tile_size: int) -> torch.Tensor:
    """``[C, H, W]`` (H, W multiples of ``tile_size``) → ``[rows·cols, C, tile, tile]`` in row-major order."""
    c, h, w = image.shape
    assert h % tile_size == 0 and w % tile_size == 0, f"Image size {h}x{w} is not divisible by tile size {tile_size}"
    rows, cols = h // tile_size, w // tile_size
    return image.reshape(c, rows, tile_size, cols, tile_size).permute(1, 3, 0, 2, 4).reshape(rows * cols, c, tile_size, tile_size).contiguous()
