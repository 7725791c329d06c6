from .attention import MultiHeadAttention
from .attention_utils import create_block_causal_mask, packed_block_causal_mask
from .classifier import classifier_model
from .common_utils import (
    delete_kv_caches,
    disable_kv_cache,
    local_kv_cache,
    reparametrize_as_dtype_state_dict_post_hook,
    slice_str_to_array,
)
from .embedding_utils import resize_token_embeddings
from .feed_forward import FeedForward
from .kv_cache import KVCache
from .layer_norm import Fp32LayerNorm
from .linear import Linear
from .low_precision import FrozenNF4Linear
from .position_embeddings import (
    HalfSplitRotaryPositionalEmbeddings,
    Llama3ScaledRoPE,
    Llama4ScaledRoPE,
    Phi3RotaryPositionalEmbeddings,
    Qwen2RotaryPositionalEmbeddings,
    RotaryPositionalEmbeddings,
    VisionRotaryPositionalEmbeddings,
)
from .rms_norm import RMSNorm, rms_norm
from .tanh_gate import TanhGate
from .tied_linear import TiedLinear
from .transformer import TransformerCrossAttentionLayer, TransformerDecoder, TransformerSelfAttentionLayer
from .layer_dropout import LayerDropout, ModuleLayerDropoutWrapper, ScaleType, get_scale, prepare_layer_dropout
from .vq_embeddings import VectorQuantizedEmbeddings
from .vision_transformer import CLSEmbedding, CLSProjection, PatchEmbedding, VisionTransformer

__all__ = [
    "MultiHeadAttention",
    "create_block_causal_mask",
    "packed_block_causal_mask",
    "LayerDropout",
    "ModuleLayerDropoutWrapper",
    "ScaleType",
    "get_scale",
    "prepare_layer_dropout",
    "VectorQuantizedEmbeddings",
    "VisionTransformer",
    "CLSEmbedding",
    "CLSProjection",
    "PatchEmbedding",
    "TanhGate",
    "FeedForward",
    "FrozenNF4Linear",
    "KVCache",
    "Linear",
    "RotaryPositionalEmbeddings",
    "VisionRotaryPositionalEmbeddings",
    "Llama3ScaledRoPE",
    "Llama4ScaledRoPE",
    "HalfSplitRotaryPositionalEmbeddings",
    "Qwen2RotaryPositionalEmbeddings",
    "Phi3RotaryPositionalEmbeddings",
    "RMSNorm",
    "rms_norm",
    "TiedLinear",
    "Fp32LayerNorm",
    "TransformerDecoder",
    "TransformerSelfAttentionLayer",
    "TransformerCrossAttentionLayer",
    "reparametrize_as_dtype_state_dict_post_hook",
    "delete_kv_caches",
    "disable_kv_cache",
    "local_kv_cache",
    "slice_str_to_array",
    "classifier_model",
    "resize_token_embeddings",
]
