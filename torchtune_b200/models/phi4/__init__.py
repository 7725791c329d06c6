"""Phi-4 14B on the Phi-3 architecture (parity: torchtune/models/phi4/_model_builders.py)."""
from typing import Optional

from .._family import lora_preset, preset, qlora_preset
from ..phi3 import lora_phi3, phi3

_C = dict(vocab_size=100_352, num_layers=40, num_heads=40, num_kv_heads=10, embed_dim=5120, intermediate_dim=17920, max_seq_len=16384, attn_dropout=0.0, norm_eps=1e-5)
phi4_14b = preset(phi3, "phi4_14b", "Phi-4 14B.", **_C)
lora_phi4_14b = lora_preset(lora_phi3, "lora_phi4_14b", "Phi-4 14B with adapters.", **_C)
qlora_phi4_14b = qlora_preset(lora_phi4_14b, "qlora_phi4_14b")


def phi4_tokenizer(vocab_path: str = None, merges_path: str = None, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import Phi4Tokenizer

    special = parse_hf_tokenizer_json(special_tokens_path) if special_tokens_path is not None else None
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Phi4Tokenizer(vocab_path=vocab_path, merges_path=merges_path, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type)
