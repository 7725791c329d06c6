"""GSM8K builders under the module path the reference uses (torchtune/dev/grpo/gsm8k.py); the code lives in
:mod:`torchtune_b200.dev.grpo.data`."""
from .data import gsm8k_dataset, gsm8k_sft, normalize_gsm, sft_gsm_transform

__all__ = ["gsm8k_dataset", "gsm8k_sft", "normalize_gsm", "sft_gsm_transform"]
