"""Image preprocessing for tiled CLIP encoders (parity: torchtune/models/clip/_transform.py:24-190)."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Tuple

import torch

from ...modules.transforms.vision_utils import find_supported_resolutions, get_canvas_best_fit, resize_with_pad, tile_crop


def to_float_image(image: Any, dtype: torch.dtype) -> torch.Tensor:
    """PIL image / uint8 or float tensor → float ``[C, H, W]`` in ``[0, 1]``."""
    if not isinstance(image, torch.Tensor):
        import numpy as np

        if getattr(image, "mode", "RGB") != "RGB":
            image = image.convert("RGB")
        image = torch.from_numpy(np.asarray(image).copy()).permute(2, 0, 1)
    if image.dtype == torch.uint8:
        return image.to(dtype) / 255.0 if dtype.is_floating_point else image
    return image.to(dtype)


class CLIPImageTransform:
    """Pick the canvas (a grid of at most ``max_num_tiles`` tiles) that fits the image with the
    least distortion, resize onto it preserving aspect ratio (zero-padded bottom/right),
    normalise, and cut into ``tile_size`` tiles.  Adds ``image`` ``[n_tiles, C, tile, tile]`` and
    ``aspect_ratio`` ``[2]`` (tile rows, tile columns) to the sample."""

    def __init__(self, *, image_mean: Optional[List[float]] = None, image_std: Optional[List[float]] = None, possible_resolutions: Optional[List[Tuple[int, int]]] = None,
                 tile_size: int = 224, max_num_tiles: Optional[int] = 4, dtype: torch.dtype = torch.bfloat16, resample: str = "bilinear", resize_to_max_canvas: bool = False) -> None:
        assert possible_resolutions is not None or max_num_tiles is not None, f"Either possible_resolutions or max_num_tiles must be given. Got {possible_resolutions=} and {max_num_tiles=}"
        if not possible_resolutions and max_num_tiles:
            possible_resolutions = find_supported_resolutions(max_num_tiles=max_num_tiles, tile_size=tile_size)
        self.possible_resolutions = torch.tensor(possible_resolutions).reshape(-1, 2)
        self.resize_to_max_canvas = resize_to_max_canvas
        assert (image_mean is None) == (image_std is None), f"Need to provide both or none of image_mean and image_std. Got {image_mean=} and {image_std=}"
        self.mean, self.std = image_mean, image_std
        self.max_size = None if resize_to_max_canvas else tile_size
        self.dtype, self.resample, self.tile_size = dtype, resample, tile_size

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        image = to_float_image(sample["image"], torch.float32)
        canvas = get_canvas_best_fit(image, self.possible_resolutions, self.resize_to_max_canvas)
        image = resize_with_pad(image, canvas, self.resample, self.max_size)
        if self.mean:
            mean = torch.tensor(self.mean, dtype=image.dtype).view(-1, 1, 1)
            std = torch.tensor(self.std, dtype=image.dtype).view(-1, 1, 1)
            image = (image - mean) / std
        sample = dict(sample)
        sample["image"] = tile_crop(image.to(self.dtype), self.tile_size)
        sample["aspect_ratio"] = torch.tensor(canvas).reshape(-1) // self.tile_size
        return sample
