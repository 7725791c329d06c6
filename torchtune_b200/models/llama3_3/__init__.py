"""Llama 3.3 70B: the Llama-3.1 70B architecture under its own names
(parity: torchtune/models/llama3_3/_model_builders.py:17-31)."""
from ..llama3_1 import llama3_1_70b as llama3_3_70b
from ..llama3_1 import lora_llama3_1_70b as lora_llama3_3_70b
from ..llama3_1 import qlora_llama3_1_70b as qlora_llama3_3_70b

__all__ = ["llama3_3_70b", "lora_llama3_3_70b", "qlora_llama3_3_70b"]
