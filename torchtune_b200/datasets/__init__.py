from . import multimodal
from ._builders import (
    alpaca_cleaned_dataset,
    alpaca_dataset,
    chat_dataset,
    cnn_dailymail_articles_dataset,
    grammar_dataset,
    hh_rlhf_helpful_dataset,
    instruct_dataset,
    samsum_dataset,
    slimorca_dataset,
    stack_exchange_paired_dataset,
    wikitext_dataset,
)
from ._concat import ConcatDataset
from ._interleaved import InterleavedDataset
from ._packed import PackedDataset
from ._preference import PreferenceDataset, preference_dataset
from ._sft import SFTDataset, SFTTransform
from ._synthetic import (
    SyntheticPackedDataset,
    SyntheticPreferenceDataset,
    SyntheticSFTDataset,
    synthetic_packed_dataset,
    synthetic_preference_dataset,
    synthetic_sft_dataset,
)
from ._text_completion import TextCompletionDataset, text_completion_dataset

__all__ = [
    "InterleavedDataset",
    "multimodal",
    "alpaca_cleaned_dataset",
    "alpaca_dataset",
    "chat_dataset",
    "cnn_dailymail_articles_dataset",
    "ConcatDataset",
    "grammar_dataset",
    "hh_rlhf_helpful_dataset",
    "instruct_dataset",
    "preference_dataset",
    "samsum_dataset",
    "SFTDataset",
    "SFTTransform",
    "slimorca_dataset",
    "PackedDataset",
    "PreferenceDataset",
    "stack_exchange_paired_dataset",
    "text_completion_dataset",
    "TextCompletionDataset",
    "wikitext_dataset",
    "SyntheticPackedDataset",
    "SyntheticPreferenceDataset",
    "SyntheticSFTDataset",
    "synthetic_packed_dataset",
    "synthetic_preference_dataset",
    "synthetic_sft_dataset",
]
