"""Building blocks for attaching new modalities to a pre-trained decoder
(parity: torchtune/modules/model_fusion/_fusion_layers.py:11-290, _fusion_utils.py:12-60).

A *fusion* module is one whose parameters did not exist in the pre-trained decoder.  Modules
declare them through ``fusion_params()``; :func:`get_fusion_params` collects them so recipes can
train the new parts while the original weights stay frozen.  The wrappers rewrite state-dict
keys so that the wrapped decoder still loads the original checkpoint unchanged.
"""
from __future__ import annotations

from typing import Dict, List

import torch
from torch import nn


def register_fusion_module(module: nn.Module) -> None:
    """Mark every parameter of ``module`` as a fusion parameter."""

    def fusion_params(self) -> List[str]:
        return [name for name, _ in self.named_parameters()]

    module.fusion_params = fusion_params.__get__(module)


def get_fusion_params(model: nn.Module) -> Dict[str, nn.Parameter]:
    """Fully-qualified name → parameter for everything declared by a ``fusion_params()`` method."""
    out: Dict[str, nn.Parameter] = {}
    for prefix, mod in model.named_modules():
        declare = getattr(mod, "fusion_params", None)
        if not callable(declare):
            continue
        own = dict(mod.named_parameters(recurse=True))
        names = list(declare())
        for name in names:
            if name not in own:
                raise AssertionError(f"Invalid fusion parameter {name!r} declared by {type(mod).__name__}; module parameters: {sorted(own)}")
            out[f"{prefix}.{name}" if prefix else name] = own[name]
    return out


class FusionLayer(nn.Module):
    """Runs a new ``fusion_layer`` before (or after) an original ``layer``.  In the state dict the
    original layer's keys keep their old names (no ``layer.`` prefix); only ``fusion_layer.*`` is new."""

    def __init__(self, layer: nn.Module, fusion_layer: nn.Module, fusion_first: bool = True):
        super().__init__()
        self.layer, self.fusion_layer, self.fusion_first = layer, fusion_layer, fusion_first
        self._register_state_dict_hook(FusionLayer._flatten_keys)
        self._register_load_state_dict_pre_hook(FusionLayer._nest_keys, with_module=True)

    def _flatten_keys(self, state_dict, prefix, *args, **kwargs):
        for key in [k for k in state_dict if k.startswith(prefix + "layer.")]:
            state_dict[prefix + key[len(prefix) + len("layer.") :]] = state_dict.pop(key)

    def _nest_keys(self, state_dict, prefix, *args, **kwargs):
        for key in [k for k in state_dict if k.startswith(prefix)]:
            local = key[len(prefix) :]
            if not local.startswith("fusion_layer") and not local.startswith("layer."):
                state_dict[prefix + "layer." + local] = state_dict.pop(key)

    def setup_caches(self, batch_size: int, dtype: torch.dtype, *, encoder_max_seq_len: int, decoder_max_seq_len: int) -> None:
        for m in (self.layer, self.fusion_layer):
            m.setup_caches(batch_size, dtype, encoder_max_seq_len=encoder_max_seq_len, decoder_max_seq_len=decoder_max_seq_len)

    def caches_are_setup(self) -> bool:
        return self.layer.caches_are_setup()

    def caches_are_enabled(self) -> bool:
        return self.layer.caches_are_enabled()

    def reset_cache(self) -> None:
        self.layer.reset_cache()
        self.fusion_layer.reset_cache()

    def fusion_params(self) -> List[str]:
        return [f"fusion_layer.{k}" for k, _ in self.fusion_layer.named_parameters()]

    def forward(self, x: torch.Tensor, **kwargs) -> torch.Tensor:
        if self.fusion_first:
            return self.layer(self.fusion_layer(x, **kwargs), **kwargs)
        return self.fusion_layer(self.layer(x, **kwargs), **kwargs)


class FusionEmbedding(nn.Module):
    """Token embedding extended by ``fusion_vocab_size`` new rows kept in a separate (trainable)
    table; ids ``>= vocab_size`` index the new table.  The original table is saved as ``weight``."""

    def __init__(self, vocab_size: int, fusion_vocab_size: int, embed_dim: int) -> None:
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, embed_dim)
        self.fusion_embedding = nn.Embedding(fusion_vocab_size, embed_dim)
        self.dim = embed_dim
        self.num_embeddings = vocab_size + fusion_vocab_size
        self._register_state_dict_hook(FusionEmbedding._save_hook)
        self._register_load_state_dict_pre_hook(FusionEmbedding._load_hook, with_module=True)

    @property
    def embedding_dim(self) -> int:
        return self.dim

    def _save_hook(self, destination, prefix, keep_vars):
        destination[prefix + "weight"] = destination.pop(prefix + "embedding.weight")

    def _load_hook(self, state_dict, prefix, *args, **kwargs):
        if prefix + "weight" in state_dict:
            state_dict[prefix + "embedding.weight"] = state_dict.pop(prefix + "weight")

    def fusion_params(self) -> List[str]:
        return ["fusion_embedding.weight"]

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        n = self.embedding.num_embeddings
        is_base = input < n
        base = self.embedding(input.clamp_max(n - 1))
        extra = self.fusion_embedding((input - n).clamp_min(0))
        return torch.where(is_base.unsqueeze(-1), base, extra.to(base.dtype))
