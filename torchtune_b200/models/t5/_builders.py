"""T5 encoder builders, tokenizer and HF converter
(parity: torchtune/models/t5/_component_builders.py, _model_builders.py, _tokenizer.py, _convert_weights.py)."""
from __future__ import annotations

import re
from typing import Any, Dict, List

import torch
from torch import nn

from ...modules import FeedForward, Linear, RMSNorm
from ...modules.transforms.tokenizers import SentencePieceBaseTokenizer
from ._encoder import T5Encoder, T5EncoderLayer, T5EncoderSelfAttention


def t5_encoder(embed_dim: int, mlp_dim: int, num_heads: int, head_dim: int, num_layers: int, rel_pos_num_buckets: int, rel_pos_max_dist: int, vocab_size: int, norm_eps: float, max_seq_len: int) -> T5Encoder:
    """The gate uses the tanh form of GELU, the activation the v1.1 checkpoints were trained with (``gelu_new`` in their published
    configuration); the reference builds the erf form (torchtune/models/t5/_component_builders.py:70), which differs by less than
    1e-3 per activation."""
    layers = []
    for _ in range(num_layers):
        attn = T5EncoderSelfAttention(embed_dim, num_heads, head_dim, *(Linear(embed_dim, embed_dim, bias=False) for _ in range(4)))
        mlp = FeedForward(gate_proj=Linear(embed_dim, mlp_dim, bias=False), down_proj=Linear(mlp_dim, embed_dim, bias=False), up_proj=Linear(embed_dim, mlp_dim, bias=False), activation=nn.GELU(approximate="tanh"))
        layers.append(T5EncoderLayer(attn, mlp, RMSNorm(embed_dim, eps=norm_eps), RMSNorm(embed_dim, eps=norm_eps)))
    return T5Encoder(token_embedding=nn.Embedding(vocab_size, embed_dim), layers=layers, final_norm=RMSNorm(embed_dim, eps=norm_eps), num_heads=num_heads,
                     rel_pos_num_buckets=rel_pos_num_buckets, rel_pos_max_dist=rel_pos_max_dist, max_seq_len=max_seq_len)


def t5_v1_1_xxl_encoder(max_seq_len: int = 512) -> T5Encoder:
    """Encoder of T5 v1.1 XXL: 24 layers, width 4096, 64 heads of 64, gated-GELU MLP 10240."""
    return t5_encoder(embed_dim=4096, mlp_dim=10240, num_heads=64, head_dim=64, num_layers=24, rel_pos_num_buckets=32, rel_pos_max_dist=128, vocab_size=32128, norm_eps=1e-6, max_seq_len=max_seq_len)


class T5Tokenizer(SentencePieceBaseTokenizer):
    """SentencePiece text → ids with EOS appended (no BOS), truncated to ``max_seq_len``."""

    def __init__(self, path: str, max_seq_len: int = 512, truncate: bool = True):
        super().__init__(path)
        self.max_seq_len, self.truncate = max_seq_len, truncate

    def encode(self, text: str) -> List[int]:
        tokens = super().encode(text, add_bos=False, add_eos=True, trim_leading_whitespace=False, prefix=None)
        if len(tokens) > self.max_seq_len:
            assert self.truncate, "Tokenized text is larger than the maximum sequence length but truncate is set to False."
            tokens = tokens[: self.max_seq_len]
            tokens[-1] = self.eos_id
        return tokens

    def __call__(self, sample: Dict[str, Any], inference: bool = False) -> Dict[str, Any]:
        sample["tokens"] = self.encode(sample.pop("text"))
        return sample


def t5_tokenizer(path: str, max_seq_len: int = 512, truncate: bool = True) -> T5Tokenizer:
    return T5Tokenizer(path, max_seq_len=max_seq_len, truncate=truncate)


_BLOCK = re.compile(r"^encoder\.block\.(\d+)\.layer\.(\d)\.(.+)$")
_SUB = {
    ("0", "SelfAttention.q.weight"): "attn.q_proj.weight", ("0", "SelfAttention.k.weight"): "attn.k_proj.weight", ("0", "SelfAttention.v.weight"): "attn.v_proj.weight",
    ("0", "SelfAttention.o.weight"): "attn.output_proj.weight", ("0", "layer_norm.weight"): "sa_norm.scale",
    ("1", "DenseReluDense.wi_0.weight"): "mlp.w1.weight", ("1", "DenseReluDense.wo.weight"): "mlp.w2.weight", ("1", "DenseReluDense.wi_1.weight"): "mlp.w3.weight", ("1", "layer_norm.weight"): "mlp_norm.scale",
}


def t5_encoder_hf_to_tune(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Encoder half of an HF T5 checkpoint; decoder weights and the (tied) ``shared`` / ``lm_head`` are ignored."""
    out: Dict[str, torch.Tensor] = {}
    for key, value in state_dict.items():
        if key.startswith("decoder.") or key in ("shared.weight", "lm_head.weight"):
            continue
        if key == "encoder.embed_tokens.weight":
            out["token_embedding.weight"] = value
        elif key == "encoder.final_layer_norm.weight":
            out["final_norm.scale"] = value
        else:
            m = _BLOCK.match(key)
            if m is None:
                raise KeyError(f'Error converting the state dict. Found unexpected key: "{key}".')
            block, sub, rest = m.groups()
            if rest == "SelfAttention.relative_attention_bias.weight":
                out["relative_position_bias.embedding.weight"] = value  # only block 0 carries it
            else:
                out[f"layers.{block}.{_SUB[(sub, rest)]}"] = value
    return out
