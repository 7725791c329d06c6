"""Qwen2 (parity: torchtune/models/qwen2/*): q/k/v biases, half-split RoPE with base 1e6,
small sizes tie the output projection to the embeddings."""
from typing import Optional

from ...modules import Qwen2RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset
from .._generic import component_builders, layer_builders
from ._convert_weights import qwen2_hf_to_tune, qwen2_tune_to_hf  # noqa: F401


def _arch(vocab_size: int, num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, head_dim: Optional[int] = None, attn_dropout: float = 0.0, norm_eps: float = 1e-5, rope_base: float = 1_000_000.0, tie_word_embeddings: bool = False) -> DecoderArch:
    return DecoderArch(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, intermediate_dim=intermediate_dim, head_dim=head_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, qkv_bias=True, tie_embeddings=tie_word_embeddings, rope=lambda hd, msl: Qwen2RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base))


qwen2, lora_qwen2 = component_builders("qwen2", _arch, "Qwen2 decoder: GQA with q/k/v bias, SwiGLU, RMSNorm, half-split RoPE.")
qwen2_mlp, lora_qwen2_self_attention, lora_qwen2_mlp = layer_builders(_arch)

_C = dict(max_seq_len=32768, attn_dropout=0.0, norm_eps=1e-6, rope_base=1_000_000.0)
SIZES = {
    "0_5b": dict(vocab_size=151936, num_layers=24, num_heads=14, num_kv_heads=2, embed_dim=896, intermediate_dim=4864, tie_word_embeddings=True),
    "1_5b": dict(vocab_size=151936, num_layers=28, num_heads=12, num_kv_heads=2, embed_dim=1536, intermediate_dim=8960, tie_word_embeddings=True),
    "7b": dict(vocab_size=152064, num_layers=28, num_heads=28, num_kv_heads=4, embed_dim=3584, intermediate_dim=18944),
}
for _n, _s in SIZES.items():
    globals()[f"qwen2_{_n}"] = preset(qwen2, f"qwen2_{_n}", f"Qwen2 {_n.replace('_', '.')}.", **_C, **_s)
    globals()[f"lora_qwen2_{_n}"] = lora_preset(lora_qwen2, f"lora_qwen2_{_n}", f"Qwen2 {_n.replace('_', '.')} with adapters.", **_C, **_s)


def qwen2_tokenizer(path: str, merges_file: str, special_tokens_path: Optional[str] = None, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right", **kwargs):
    from ...data._prompt_templates import _get_prompt_template
    from ...modules.transforms.tokenizers import parse_hf_tokenizer_json
    from ._tokenizer import QWEN2_SPECIAL_TOKENS, Qwen2Tokenizer

    special = QWEN2_SPECIAL_TOKENS if special_tokens_path is None else parse_hf_tokenizer_json(special_tokens_path)
    template = _get_prompt_template(prompt_template) if prompt_template is not None else None
    return Qwen2Tokenizer(path=path, merges_file=merges_file, special_tokens=special, max_seq_len=max_seq_len, prompt_template=template, truncation_type=truncation_type, **kwargs)


def __getattr__(name):
    # tokenizer classes are imported on first use (they pull in sentencepiece / regex tables)
    if name == "Qwen2Tokenizer":
        from ._tokenizer import Qwen2Tokenizer

        return Qwen2Tokenizer
    raise AttributeError(name)
