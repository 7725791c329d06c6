"""SmolLM2 135M / 360M / 1.7B — Llama-3.2-style decoders with a 49k vocabulary
(parity: torchtune/models/smol/_component_builders.py, _model_builders.py)."""
from ...modules import TransformerDecoder
from ..llama3_2 import llama3_2


def smollm2(num_layers: int, num_heads: int, num_kv_heads: int, embed_dim: int, intermediate_dim: int, max_seq_len: int = 8192, vocab_size: int = 49152, attn_dropout: float = 0.0, rope_base: int = 100000, norm_eps: float = 1e-5, scale_factor: int = 32, tie_word_embeddings: bool = True) -> TransformerDecoder:
    return llama3_2(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, num_kv_heads=num_kv_heads, embed_dim=embed_dim, max_seq_len=max_seq_len, attn_dropout=attn_dropout, rope_base=rope_base, intermediate_dim=intermediate_dim, norm_eps=norm_eps, scale_factor=scale_factor, tie_word_embeddings=tie_word_embeddings)


def smollm2_135m() -> TransformerDecoder:
    return smollm2(30, 9, 3, 576, 1536)


def smollm2_360m() -> TransformerDecoder:
    return smollm2(32, 15, 5, 960, 2560)


def smollm2_1_7b() -> TransformerDecoder:
    return smollm2(24, 32, 32, 2048, 8192, rope_base=130000)
