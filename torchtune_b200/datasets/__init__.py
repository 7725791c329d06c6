from ._concat import ConcatDataset
from ._synthetic import (
    SyntheticPackedDataset,
    SyntheticPreferenceDataset,
    SyntheticSFTDataset,
    synthetic_packed_dataset,
    synthetic_preference_dataset,
    synthetic_sft_dataset,
)

__all__ = [
    "ConcatDataset",
    "SyntheticPackedDataset",
    "SyntheticPreferenceDataset",
    "SyntheticSFTDataset",
    "synthetic_packed_dataset",
    "synthetic_preference_dataset",
    "synthetic_sft_dataset",
]
