"""Qwen3 (parity: torchtune/models/qwen3/*): explicit head_dim, no qkv bias, learnable per-head
RMSNorm on q and k applied *before* the half-split rotation (torchtune/models/qwen3/_attention.py:18)."""
from typing import Optional

from ...modules import Qwen2RotaryPositionalEmbeddings, RMSNorm
from .._factory import DecoderArch
from .._family import lora_preset, preset
from .._generic import component_builders, layer_builders
from ..qwen2._convert_weights import qwen3_hf_to_tune, qwen3_tune_to_hf  # noqa: F401


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, head_dim: Optional[int] = None, attn_dropout: float = 0.0, norm_eps: float = 1e-5, rope_base: float = 1_000_000.0, tie_word_embeddings: bool = False, q_proj_bias: bool = True, k_proj_bias: bool = True, v_proj_bias: bool = True, q_norm: bool = False, k_norm: bool = False) -> DecoderArch:
    if q_norm != k_norm:
        raise ValueError("q_norm and k_norm must be enabled together")
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, head_dim=head_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, qkv_bias=q_proj_bias and k_proj_bias and v_proj_bias, tie_embeddings=tie_word_embeddings, qk_norm=(lambda hd, eps: RMSNorm(hd, eps=eps)) if q_norm else None, qk_norm_before_rope=True, rope=lambda hd, msl: Qwen2RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


qwen3, lora_qwen3 = component_builders("qwen3", _arch, "Qwen3 decoder: GQA with per-head q/k RMSNorm before RoPE, SwiGLU, RMSNorm.")
qwen3_mlp, lora_qwen3_self_attention, lora_qwen3_mlp = layer_builders(_arch)

_B = dict(vocab_size=151936, head_dim=128, attn_dropout=0.0, norm_eps=1e-6, rope_base=1_000_000.0, q_proj_bias=False, k_proj_bias=False, v_proj_bias=False, q_norm=True, k_norm=True)
_ARCHS = {
    "0_6b": dict(num_layers=28, num_heads=16, num_kv_heads=8, embed_dim=1024, intermediate_dim=3072, tie_word_embeddings=True),
    "1_7b": dict(num_layers=28, num_heads=16, num_kv_heads=8, embed_dim=2048, intermediate_dim=6144, tie_word_embeddings=True),
    "4b": dict(num_layers=36, num_heads=32, num_kv_heads=8, embed_dim=2560, intermediate_dim=9728, tie_word_embeddings=True),
    "8b": dict(num_layers=36, num_heads=32, num_kv_heads=8, embed_dim=4096, intermediate_dim=12288),
    "14b": dict(num_layers=40, num_heads=40, num_kv_heads=8, embed_dim=5120, intermediate_dim=17408),
}
for _n, _s in _ARCHS.items():
    for _variant, _msl in (("base", 32768), ("instruct", 40960)):
        _name = f"qwen3_{_n}_{_variant}"
        globals()[_name] = preset(qwen3, _name, f"Qwen3 {_n} ({_variant}).", max_seq_len=_msl, **_B, **_s)
        globals()[f"lora_{_name}"] = lora_preset(lora_qwen3, f"lora_{_name}", f"Qwen3 {_n} ({_variant}) with adapters.", max_seq_len=_msl, **_B, **_s)
_S32 = dict(num_layers=64, num_heads=64, num_kv_heads=8, embed_dim=5120, intermediate_dim=25600, max_seq_len=40960)
qwen3_32b = preset(qwen3, "qwen3_32b", "Qwen3 32B.", **_B, **_S32)
lora_qwen3_32b = lora_preset(lora_qwen3, "lora_qwen3_32b", "Qwen3 32B with adapters.", **_B, **_S32)


def qwen3_tokenizer(path: str, merges_file: str, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right", **kwargs):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import QWEN3_SPECIAL_TOKENS, Qwen3Tokenizer

    special = QWEN3_SPECIAL_TOKENS if special_tokens_path is None else parse_hf_tokenizer_json(special_tokens_path)
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Qwen3Tokenizer(path=path, merges_file=merges_file, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type, **kwargs)
