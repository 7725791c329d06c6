from ._utils import (
    LORA_ATTN_MODULES,
    AdapterModule,
    disable_adapter,
    get_adapter_params,
    get_adapter_state_dict,
    get_lora_module_names,
    get_merged_lora_ckpt,
    set_trainable_params,
    validate_missing_and_unexpected_for_lora,
)
from .dora import DoRALinear
from .lora import LoRALinear, QATLoRALinear, TrainableParams

__all__ = [
    "AdapterModule",
    "DoRALinear",
    "LoRALinear",
    "QATLoRALinear",
    "TrainableParams",
    "LORA_ATTN_MODULES",
    "disable_adapter",
    "get_adapter_params",
    "get_adapter_state_dict",
    "get_lora_module_names",
    "get_merged_lora_ckpt",
    "set_trainable_params",
    "validate_missing_and_unexpected_for_lora",
]
