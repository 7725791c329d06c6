"""Shared test utilities."""
import json
import re
import runpy
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

from torchtune_b200.models.convert_weights import tune_to_hf

TINY = dict(vocab_size=1024, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=256, max_seq_len=256, intermediate_dim=768, norm_eps=1e-5, rope_base=500000)


def fixed_init_(model: torch.nn.Module, std: float = 0.02, seed: int = 0) -> None:
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            if p.dim() == 1 and ("norm" in name or "scale" in name):
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g) * std)


def write_tiny_hf_checkpoint(path: Path, arch=TINY, seed: int = 0, dtype=torch.float32, builder=None) -> dict:
    from torchtune_b200.models.llama3_1 import llama3_1

    path.mkdir(parents=True, exist_ok=True)
    model = (builder or llama3_1)(**arch)
    fixed_init_(model, seed=seed)
    sd = {k: v.to(dtype) for k, v in model.state_dict().items()}
    hf = tune_to_hf(sd, num_heads=arch["num_heads"], num_kv_heads=arch["num_kv_heads"], dim=arch["embed_dim"])
    save_file({k: v.contiguous() for k, v in hf.items()}, str(path / "model-00001-of-00001.safetensors"))
    (path / "config.json").write_text(
        json.dumps(
            {
                "hidden_size": arch["embed_dim"],
                "num_attention_heads": arch["num_heads"],
                "num_key_value_heads": arch["num_kv_heads"],
                "vocab_size": arch["vocab_size"],
            }
        )
    )
    return sd


def run_tune(tune_path: str, argv: str, monkeypatch) -> None:
    monkeypatch.setattr(sys, "argv", ["tune"] + argv.split())
    try:
        runpy.run_path(tune_path, run_name="__main__")
    except SystemExit as exc:
        assert exc.code in (0, None), f"tune exited with {exc.code}"


def read_losses(log_file: Path):
    return [float(m) for m in re.findall(r"loss:(\S+)", Path(log_file).read_text())]


def tiny_early_fusion_llama4():
    """A Llama-4-shaped early-fusion model small enough for CPU tests (configs name it as ``helpers.tiny_early_fusion_llama4``)."""
    from torchtune_b200.models.llama4 import llama4_decoder, llama4_vision_encoder
    from torchtune_b200.modules.model_fusion import EarlyFusionModel

    decoder = llama4_decoder(vocab_size=72, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, hidden_dim=48, max_seq_len=64, num_experts=4, experts_per_token=1, rope_base=10000,
                             skip_rope_interval=2, attention_chunk_size=16)
    tower = llama4_vision_encoder(patch_size=4, num_heads=4, clip_embed_dim=32, clip_num_layers=1, clip_hidden_states=None, projection_embed_dim=48, decoder_embed_dim=32, tile_size=16,
                                  max_num_tiles=1, in_channels=3)
    return EarlyFusionModel(decoder, encoders={"vision": tower}, encoder_tokens={"vision": 70})
