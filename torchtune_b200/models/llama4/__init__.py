"""Llama 4 (mixture-of-experts decoder with early-fused vision; parity: torchtune/models/llama4/__init__.py)."""
from ...modules.position_embeddings import Llama4ScaledRoPE
from ._chunked_attention import get_chunked_attention_mask
from ._component_builders import llama4_decoder, llama4_mlp, llama4_moe, llama4_vision_encoder, llama4_vision_projection_head, lora_llama4_decoder, lora_llama4_moe, lora_llama4_vision_encoder, lora_llama4_vision_projection_head
from ._convert_weights import llama4_hf_to_tune, llama4_tune_to_hf
from ._encoder import Llama4VisionEncoder, Llama4VisionProjectionHead
from ._model_builders import llama4_maverick_17b_128e, llama4_scout_17b_16e, llama4_transform, lora_llama4_maverick_17b_128e, lora_llama4_scout_17b_16e
from ._tokenizer import LLAMA4_SPECIAL_TOKENS, Llama4Tokenizer
from ._transform import Llama4Transform
from ._parallelism import decoder_only_tp_inference_plan, decoder_only_tp_plan, decoder_only_tp_training_plan

__all__ = [
    "lora_llama4_vision_encoder",
    "lora_llama4_vision_projection_head",
    "decoder_only_tp_plan",
    "LLAMA4_SPECIAL_TOKENS",
    "Llama4ScaledRoPE",
    "Llama4Tokenizer",
    "Llama4Transform",
    "Llama4VisionEncoder",
    "Llama4VisionProjectionHead",
    "get_chunked_attention_mask",
    "llama4_decoder",
    "llama4_hf_to_tune",
    "llama4_maverick_17b_128e",
    "llama4_mlp",
    "llama4_moe",
    "llama4_scout_17b_16e",
    "llama4_transform",
    "llama4_tune_to_hf",
    "llama4_vision_encoder",
    "llama4_vision_projection_head",
    "lora_llama4_decoder",
    "lora_llama4_maverick_17b_128e",
    "lora_llama4_moe",
    "lora_llama4_scout_17b_16e",
]
