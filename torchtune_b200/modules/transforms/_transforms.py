"""Sample transforms (parity: torchtune/modules/transforms/_transforms.py:12-179)."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Protocol

import torch


class Transform(Protocol):
    """Anything that maps a sample dict to a sample dict."""

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]: ...


class VisionCrossAttentionMask(Transform):
    """Builds, per image, the boolean ``[text_len, image_tokens]`` mask saying which text
    positions may attend to that image: tokens from an image token up to (not including) the
    next one attend to it; consecutive image tokens share the span of the last of the run;
    the final image is visible until the end of the sequence."""

    def __init__(self, tile_size: int, patch_size: int, image_token_id: int, max_num_tiles: Optional[int] = None):
        grid = tile_size // patch_size
        self.patches_per_tile = grid * grid
        self.image_token_id = image_token_id
        self.max_num_tiles = max_num_tiles

    def _get_image_attention_intervals(self, tokens: List[int]) -> List[List[int]]:
        end = len(tokens)
        locs = [i for i, t in enumerate(tokens) if t == self.image_token_id]
        if not locs:
            return []
        intervals: List[List[int]] = []
        for i, start in enumerate(locs):
            stop = locs[i + 1] if i + 1 < len(locs) else end
            intervals.append([start, stop])
        # a run of adjacent image tokens shares the interval end of the run's last member
        for i in range(len(intervals) - 2, -1, -1):
            if intervals[i][1] == intervals[i][0] + 1 and intervals[i + 1][0] == intervals[i][1]:
                intervals[i][1] = intervals[i + 1][1]
        return intervals

    def __call__(self, sample: Mapping[str, Any], inference: bool = False) -> Mapping[str, Any]:
        tokens, images = sample["tokens"], sample["encoder_input"]["images"]
        intervals = self._get_image_attention_intervals(tokens)
        if len(intervals) != len(images):
            raise RuntimeError(f"The number of image tokens ({len(intervals)}) does not match the number of images ({len(images)}).")
        masks = []
        for (start, stop), image in zip(intervals, images):
            n_tiles = image.shape[0]
            tokens_per_image = n_tiles * (self.patches_per_tile + 1)  # +1: CLS token per tile
            pad_tiles = self.max_num_tiles if (inference and self.max_num_tiles is not None) else n_tiles
            m = torch.zeros(len(tokens), pad_tiles * (self.patches_per_tile + 1), dtype=torch.bool)
            m[start:stop, :tokens_per_image] = True
            masks.append(m)
        sample.update({"encoder_mask": masks})
        return sample
