"""Gemma 2B / 7B (parity: torchtune/models/gemma/*): tied embeddings scaled by √dim,
``(1 + scale)`` RMSNorm, GELU(tanh)-gated MLP, explicit head_dim."""
from typing import Optional

from torch import nn

from ...modules import RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import component_builders, layer_builders
from ._modules import GemmaNormEmbeddings, GemmaRMSNorm, TanhSoftCapping  # noqa: F401


def _arch(vocab_size: int, num_layers: int, num_heads: int, head_dim: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, attn_dropout: float = 0.0, norm_eps: float = 1e-6, rope_base: int = 10_000) -> DecoderArch:
    return DecoderArch(
        vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len,
        intermediate_dim=intermediate_dim, head_dim=head_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, tie_embeddings=True,
        norm=lambda d, eps: GemmaRMSNorm(d, eps=eps), embedding=lambda v, d: GemmaNormEmbeddings(v, d), activation=lambda: nn.GELU(approximate="tanh"),
        rope=lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base),
    )


gemma, _lora_gemma = component_builders("gemma", _arch, "Gemma decoder.")
gemma_mlp, lora_gemma_self_attention, lora_gemma_mlp = layer_builders(_arch)


def lora_gemma(lora_attn_modules, apply_lora_to_mlp: bool = False, **kwargs):
    """Gemma with adapters (the tied output projection cannot carry one)."""
    return _lora_gemma(lora_attn_modules, apply_lora_to_mlp, False, **kwargs)


_C = dict(vocab_size=256_000, max_seq_len=8192, attn_dropout=0.0, norm_eps=1e-6)
_S = {
    "2b": dict(num_layers=18, num_heads=8, head_dim=256, num_kv_heads=1, embed_dim=2048, intermediate_dim=16384),
    "7b": dict(num_layers=28, num_heads=16, head_dim=256, num_kv_heads=16, embed_dim=3072, intermediate_dim=24576),
}
gemma_2b = preset(gemma, "gemma_2b", "Gemma 2B.", **_C, **_S["2b"])
gemma_7b = preset(gemma, "gemma_7b", "Gemma 7B.", **_C, **_S["7b"])
lora_gemma_2b = lora_preset(_lora_gemma, "lora_gemma_2b", "Gemma 2B with adapters.", **_C, **_S["2b"])
lora_gemma_7b = lora_preset(_lora_gemma, "lora_gemma_7b", "Gemma 7B with adapters.", **_C, **_S["7b"])
qlora_gemma_2b = qlora_preset(lora_gemma_2b, "qlora_gemma_2b")
qlora_gemma_7b = qlora_preset(lora_gemma_7b, "qlora_gemma_7b")


def gemma_tokenizer(path: str, max_seq_len: Optional[int] = None, prompt_template=None, truncation_type: str = "right"):
    from ...data._prompt_templates import _get_prompt_template
    from ._tokenizer import GemmaTokenizer

    return GemmaTokenizer(path=path, max_seq_len=max_seq_len, prompt_template=_get_prompt_template(prompt_template) if prompt_template is not None else None, truncation_type=truncation_type)


def __getattr__(name):
    # tokenizer classes are imported on first use (they pull in sentencepiece / regex tables)
    if name == "GemmaTokenizer":
        from ._tokenizer import GemmaTokenizer

        return GemmaTokenizer
    raise AttributeError(name)
