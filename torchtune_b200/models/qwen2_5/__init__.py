"""Qwen2.5 size presets on the Qwen2 architecture (parity: torchtune/models/qwen2_5/_model_builders.py)."""
from typing import Optional

from .._family import lora_preset, preset
from ..qwen2 import lora_qwen2, qwen2

_B = dict(attn_dropout=0.0, rope_base=1_000_000.0)
_V1, _V2 = 151936, 152064
SIZES = {
    "0_5b": dict(vocab_size=_V1, num_layers=24, num_heads=14, num_kv_heads=2, embed_dim=896, intermediate_dim=4864, max_seq_len=32768, norm_eps=1e-6, tie_word_embeddings=True),
    "1_5b_base": dict(vocab_size=_V1, num_layers=28, num_heads=12, num_kv_heads=2, embed_dim=1536, intermediate_dim=8960, max_seq_len=131072, norm_eps=1e-6, tie_word_embeddings=True),
    "1_5b_instruct": dict(vocab_size=_V1, num_layers=28, num_heads=12, num_kv_heads=2, embed_dim=1536, intermediate_dim=8960, max_seq_len=32768, norm_eps=1e-6, tie_word_embeddings=True),
    "3b": dict(vocab_size=_V1, num_layers=36, num_heads=16, num_kv_heads=2, embed_dim=2048, intermediate_dim=11008, max_seq_len=32768, norm_eps=1e-6, tie_word_embeddings=True),
    "7b_base": dict(vocab_size=_V2, num_layers=28, num_heads=28, num_kv_heads=4, embed_dim=3584, intermediate_dim=18944, max_seq_len=131072, norm_eps=1e-6),
    "7b_instruct": dict(vocab_size=_V2, num_layers=28, num_heads=28, num_kv_heads=4, embed_dim=3584, intermediate_dim=18944, max_seq_len=32768, norm_eps=1e-6),
    "14b_base": dict(vocab_size=_V2, num_layers=48, num_heads=40, num_kv_heads=8, embed_dim=5120, intermediate_dim=13824, max_seq_len=131072, norm_eps=1e-5),
    "14b_instruct": dict(vocab_size=_V2, num_layers=48, num_heads=40, num_kv_heads=8, embed_dim=5120, intermediate_dim=13824, max_seq_len=32768, norm_eps=1e-6),
    "32b_base": dict(vocab_size=_V2, num_layers=64, num_heads=40, num_kv_heads=8, embed_dim=5120, intermediate_dim=27648, max_seq_len=131072, norm_eps=1e-5),
    "32b_instruct": dict(vocab_size=_V2, num_layers=64, num_heads=40, num_kv_heads=8, embed_dim=5120, intermediate_dim=27648, max_seq_len=32768, norm_eps=1e-6),
    "72b_base": dict(vocab_size=_V2, num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, intermediate_dim=29568, max_seq_len=131072, norm_eps=1e-5),
    "72b_instruct": dict(vocab_size=_V2, num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, intermediate_dim=29568, max_seq_len=32768, norm_eps=1e-6),
}
for _n, _s in SIZES.items():
    globals()[f"qwen2_5_{_n}"] = preset(qwen2, f"qwen2_5_{_n}", f"Qwen2.5 {_n}.", **_B, **_s)
    globals()[f"lora_qwen2_5_{_n}"] = lora_preset(lora_qwen2, f"lora_qwen2_5_{_n}", f"Qwen2.5 {_n} with adapters.", **_B, **_s)


def qwen2_5_tokenizer(path: str, merges_file: str, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right", **kwargs):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import QWEN2_5_SPECIAL_TOKENS, Qwen2_5Tokenizer

    special = QWEN2_5_SPECIAL_TOKENS if special_tokens_path is None else parse_hf_tokenizer_json(special_tokens_path)
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Qwen2_5Tokenizer(path=path, merges_file=merges_file, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type, **kwargs)
