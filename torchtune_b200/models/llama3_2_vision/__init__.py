"""Llama 3.2 Vision (deep fusion of a tiled CLIP encoder into Llama 3.1 through gated
cross-attention; parity: torchtune/models/llama3_2_vision/__init__.py)."""
from ._component_builders import (
    LoRATrainable,
    llama3_2_vision_decoder,
    llama3_2_vision_encoder,
    llama3_2_vision_projection_head,
    lora_llama3_2_vision_decoder,
    lora_llama3_2_vision_encoder,
    lora_llama3_2_vision_projection_head,
)
from ._convert_weights import llama3_vision_hf_to_tune, llama3_vision_tune_to_hf
from ._encoder import Llama3VisionEncoder, Llama3VisionProjectionHead
from ._model_builders import (
    llama3_2_vision_11b,
    llama3_2_vision_90b,
    llama3_2_vision_transform,
    lora_llama3_2_vision_11b,
    lora_llama3_2_vision_90b,
    qlora_llama3_2_vision_11b,
    qlora_llama3_2_vision_90b,
)
from ._transform import Llama3VisionTransform

__all__ = [
    "LoRATrainable",
    "Llama3VisionEncoder",
    "Llama3VisionProjectionHead",
    "Llama3VisionTransform",
    "llama3_2_vision_11b",
    "llama3_2_vision_90b",
    "llama3_2_vision_decoder",
    "llama3_2_vision_encoder",
    "llama3_2_vision_projection_head",
    "llama3_2_vision_transform",
    "llama3_vision_hf_to_tune",
    "llama3_vision_tune_to_hf",
    "lora_llama3_2_vision_11b",
    "lora_llama3_2_vision_90b",
    "lora_llama3_2_vision_decoder",
    "lora_llama3_2_vision_encoder",
    "lora_llama3_2_vision_projection_head",
    "qlora_llama3_2_vision_11b",
    "qlora_llama3_2_vision_90b",
]
