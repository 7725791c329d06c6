"""Llama 3.1 size presets (parity: torchtune/models/llama3_1/_model_builders.py:20-330)."""
from .._family import lora_preset, preset, qlora_preset
from ._component_builders import llama3_1, lora_llama3_1

_COMMON = dict(vocab_size=128_256, max_seq_len=131072, attn_dropout=0.0, norm_eps=1e-5, rope_base=500_000)
_SIZES = {
    "8b": dict(num_layers=32, num_heads=32, num_kv_heads=8, embed_dim=4096, intermediate_dim=14336),
    "70b": dict(num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, intermediate_dim=28672),
    "405b": dict(num_layers=126, num_heads=128, num_kv_heads=8, embed_dim=16384, intermediate_dim=53248),
}

llama3_1_8b = preset(llama3_1, "llama3_1_8b", "Llama 3.1 8B.", **_COMMON, **_SIZES["8b"])
llama3_1_70b = preset(llama3_1, "llama3_1_70b", "Llama 3.1 70B.", **_COMMON, **_SIZES["70b"])
llama3_1_405b = preset(llama3_1, "llama3_1_405b", "Llama 3.1 405B.", **_COMMON, **_SIZES["405b"])
lora_llama3_1_8b = lora_preset(lora_llama3_1, "lora_llama3_1_8b", "Llama 3.1 8B with LoRA/DoRA adapters.", **_COMMON, **_SIZES["8b"])
lora_llama3_1_70b = lora_preset(lora_llama3_1, "lora_llama3_1_70b", "Llama 3.1 70B with LoRA/DoRA adapters.", **_COMMON, **_SIZES["70b"])
lora_llama3_1_405b = lora_preset(lora_llama3_1, "lora_llama3_1_405b", "Llama 3.1 405B with LoRA adapters.", **_COMMON, **_SIZES["405b"])
qlora_llama3_1_8b = qlora_preset(lora_llama3_1_8b, "qlora_llama3_1_8b")
qlora_llama3_1_70b = qlora_preset(lora_llama3_1_70b, "qlora_llama3_1_70b")
qlora_llama3_1_405b = qlora_preset(lora_llama3_1_405b, "qlora_llama3_1_405b")
