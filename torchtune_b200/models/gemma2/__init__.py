"""Gemma 2 (parity: torchtune/models/gemma2/*): attention-logit soft capping, sliding window on
even layers, post-attention / post-MLP norms, soft-capped final norm, optional
``query_pre_attn_scalar``.  The reference carries its own eager attention class for this
(torchtune/models/gemma2/_attention.py:19-340); here the shared attention module takes the
soft-cap, the scale and a per-layer window through the structured mask."""
from typing import Optional

from torch import nn

from ...modules import RotaryPositionalEmbeddings
from .._factory import DecoderArch
from .._family import lora_preset, preset, qlora_preset
from .._generic import component_builders, layer_builders
from ..gemma._modules import Gemma2FinalNorm, GemmaNormEmbeddings, GemmaRMSNorm, TanhSoftCapping  # noqa: F401
from ._convert_weights import gemma2_hf_to_tune, gemma2_tune_to_hf  # noqa: F401


def _arch(vocab_size: int, num_layers: int, num_heads: int, head_dim: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int, attn_dropout: float = 0.0, norm_eps: float = 1e-6, rope_base: int = 10_000, hidden_capping_value: float = 50.0, final_capping_value: float = 30.0, sliding_window_size: int = 4096, query_pre_attn_scalar: Optional[int] = None, cap_logits: bool = True) -> DecoderArch:
    # cap_logits=True: the published model (soft cap on the logits).  False: the reference's graph (cap on the final hidden state).
    return DecoderArch(
        vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len,
        intermediate_dim=intermediate_dim, head_dim=head_dim, attn_dropout=attn_dropout, norm_eps=norm_eps, tie_embeddings=True,
        norm=lambda d, eps: GemmaRMSNorm(d, eps=eps), embedding=lambda v, d: GemmaNormEmbeddings(v, d), activation=lambda: nn.GELU(approximate="tanh"),
        rope=lambda hd, msl: RotaryPositionalEmbeddings(dim=hd, max_seq_len=msl, base=rope_base),
        post_norms=True, final_norm=lambda d, eps: Gemma2FinalNorm(final_capping_value, d, eps, cap_hidden=not cap_logits),
        logit_softcap=final_capping_value if cap_logits else 0.0,
        attn_softcap=hidden_capping_value, attn_scale=(query_pre_attn_scalar or head_dim) ** -0.5,
        sliding_window=lambda idx: sliding_window_size if idx % 2 == 0 else 0,
    )


gemma2, _lora_gemma2 = component_builders("gemma2", _arch, "Gemma-2 decoder.")
gemma2_mlp, lora_gemma2_self_attention, lora_gemma2_mlp = layer_builders(_arch)


def lora_gemma2(lora_attn_modules, apply_lora_to_mlp: bool = False, **kwargs):
    return _lora_gemma2(lora_attn_modules, apply_lora_to_mlp, False, **kwargs)


# attention scores are capped at 50 and logits at 30, as in the published configuration (the reference's presets pass the two the
# other way round, torchtune/models/gemma2/_model_builders.py:38-39)
_C = dict(vocab_size=256_000, max_seq_len=8192, attn_dropout=0.0, norm_eps=1e-6, hidden_capping_value=50.0, final_capping_value=30.0, sliding_window_size=4096)
_S = {
    "2b": dict(num_layers=26, num_heads=8, head_dim=256, num_kv_heads=4, embed_dim=2304, intermediate_dim=9216),
    "9b": dict(num_layers=42, num_heads=16, head_dim=256, num_kv_heads=8, embed_dim=3584, intermediate_dim=14336),
    "27b": dict(num_layers=46, num_heads=32, head_dim=128, num_kv_heads=16, embed_dim=4608, intermediate_dim=36864, query_pre_attn_scalar=144),
}
for _n, _s in _S.items():
    globals()[f"gemma2_{_n}"] = preset(gemma2, f"gemma2_{_n}", f"Gemma-2 {_n}.", **_C, **_s)
    globals()[f"lora_gemma2_{_n}"] = lora_preset(_lora_gemma2, f"lora_gemma2_{_n}", f"Gemma-2 {_n} with adapters.", **_C, **_s)
    globals()[f"qlora_gemma2_{_n}"] = qlora_preset(globals()[f"lora_gemma2_{_n}"], f"qlora_gemma2_{_n}")

from ..gemma import gemma_tokenizer  # gemma 2 uses the gemma tokenizer


def __getattr__(name):
    if name == "GemmaTokenizer":
        from ..gemma._tokenizer import GemmaTokenizer

        return GemmaTokenizer
    raise AttributeError(name)
