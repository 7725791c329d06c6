"""Size presets instantiate on the meta device with the parameter counts of the published models."""
import importlib

import pytest
import torch

PRESETS = [
    ("llama2", "llama2_7b", 6_738_415_616), ("llama3", "llama3_8b", 8_030_261_248), ("llama3_1", "llama3_1_8b", 8_030_261_248),
    ("llama3_1", "llama3_1_70b", 70_553_706_496), ("llama3_2", "llama3_2_1b", 1_235_814_400), ("llama3_2", "llama3_2_3b", 3_212_749_824),
    ("mistral", "mistral_7b", 7_241_732_096), ("qwen2_5", "qwen2_5_7b_instruct", 7_615_616_512), ("qwen3", "qwen3_8b_instruct", 8_190_735_360),
    ("gemma", "gemma_2b", 2_506_172_416), ("gemma2", "gemma2_9b", 9_241_705_984), ("phi3", "phi3_mini", 3_821_079_552),
]


@pytest.mark.parametrize("family,builder,numel", PRESETS)
def test_preset_parameter_count(family, builder, numel):
    fn = getattr(importlib.import_module(f"torchtune_b200.models.{family}"), builder)
    with torch.device("meta"):
        model = fn()
    assert sum(p.numel() for p in model.parameters()) == numel
