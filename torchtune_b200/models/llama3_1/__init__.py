from ...modules.position_embeddings import Llama3ScaledRoPE
from ._component_builders import llama3_1, llama3_mlp, lora_llama3_1, lora_llama3_attention, lora_llama3_mlp
from ._model_builders import (
    llama3_1_405b,
    llama3_1_70b,
    llama3_1_8b,
    lora_llama3_1_405b,
    lora_llama3_1_70b,
    lora_llama3_1_8b,
    qlora_llama3_1_405b,
    qlora_llama3_1_70b,
    qlora_llama3_1_8b,
)

__all__ = [
    "llama3_1",
    "llama3_1_8b",
    "llama3_1_70b",
    "llama3_1_405b",
    "lora_llama3_1",
    "lora_llama3_1_8b",
    "lora_llama3_1_70b",
    "lora_llama3_1_405b",
    "qlora_llama3_1_8b",
    "qlora_llama3_1_70b",
    "qlora_llama3_1_405b",
    "Llama3ScaledRoPE",
    "llama3_mlp",
    "lora_llama3_attention",
    "lora_llama3_mlp",
]
