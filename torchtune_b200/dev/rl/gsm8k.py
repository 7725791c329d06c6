"""GSM8K builders under the module path the reference uses (torchtune/dev/rl/gsm8k.py:25-130); the code lives in
:mod:`torchtune_b200.dev.grpo.data`."""
from ..grpo.data import gsm8k_dataset, gsm8k_sft, normalize_gsm, sft_gsm_transform

__all__ = ["gsm8k_dataset", "gsm8k_sft", "normalize_gsm", "sft_gsm_transform"]
