from ._collate import (
    left_pad_sequence,
    padded_collate,
    padded_collate_dpo,
    padded_collate_packed,
    padded_collate_sft,
    padded_collate_tiled_images_and_mask,
)
from ._common import CROSS_ENTROPY_IGNORE_IDX

__all__ = [
    "CROSS_ENTROPY_IGNORE_IDX",
    "left_pad_sequence",
    "padded_collate",
    "padded_collate_dpo",
    "padded_collate_packed",
    "padded_collate_sft",
    "padded_collate_tiled_images_and_mask",
]
