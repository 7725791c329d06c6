"""Deep-fusion (cross-attention) and early-fusion (embedding splice) multimodal wrappers
(parity: torchtune/modules/model_fusion/_deep_fusion.py:17-215, _early_fusion.py:17-280)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch
from torch import nn

from ... import ops
from ..peft import set_trainable_params
from ._layers import get_fusion_params


class _FusionBase(nn.Module):
    decoder: nn.Module

    def set_num_output_chunks(self, num_output_chunks: int) -> None:
        self.decoder.set_num_output_chunks(num_output_chunks)

    def setup_caches(self, batch_size: int, dtype: torch.dtype, *, encoder_max_seq_len: Optional[int] = None, decoder_max_seq_len: Optional[int] = None) -> None:
        self.decoder.setup_caches(batch_size, dtype, encoder_max_seq_len=encoder_max_seq_len, decoder_max_seq_len=decoder_max_seq_len)

    def caches_are_setup(self) -> bool:
        return self.decoder.caches_are_setup()

    def caches_are_enabled(self) -> bool:
        return self.decoder.caches_are_enabled()

    def reset_caches(self) -> None:
        self.decoder.reset_caches()

    @property
    def output(self) -> nn.Module:
        return self.decoder.output

    @property
    def skip_output_layer(self) -> bool:
        return self.decoder.skip_output_layer

    @skip_output_layer.setter
    def skip_output_layer(self, skip: bool) -> None:
        self.decoder.skip_output_layer = skip

    def _freeze_except(self, trainable: set, fusion_trainable: bool) -> None:
        fusion = set(get_fusion_params(self))
        trainable = (trainable | fusion) if fusion_trainable else (trainable - fusion)
        set_trainable_params(self, trainable)


class DeepFusionModel(_FusionBase):
    """``encoder(**encoder_input)`` produces a sequence the decoder's cross-attention (fusion) layers
    attend to; ``encoder_mask`` says which text tokens see which encoder tokens."""

    def __init__(self, decoder: nn.Module, encoder: nn.Module, *, decoder_trainable: bool = False, encoder_trainable: bool = False, fusion_trainable: bool = True):
        super().__init__()
        self.decoder, self.encoder = decoder, encoder
        trainable = set()
        if encoder_trainable:
            trainable |= {f"encoder.{n}" for n, _ in encoder.named_parameters()}
        if decoder_trainable:
            trainable |= {f"decoder.{n}" for n, _ in decoder.named_parameters()}
        self._freeze_except(trainable, fusion_trainable)

    def forward(self, tokens: torch.Tensor, *, mask=None, encoder_input: Optional[Dict[str, Any]] = None, encoder_mask: Optional[torch.Tensor] = None, input_pos: Optional[torch.Tensor] = None) -> Union[torch.Tensor, List[torch.Tensor]]:
        encoded = self.encoder(**encoder_input) if encoder_input is not None else None
        return self.decoder(tokens=tokens, mask=mask, encoder_input=encoded, encoder_mask=encoder_mask, input_pos=input_pos)


class EarlyFusionModel(_FusionBase):
    """Each encoder's output embeddings replace the positions of its placeholder token in the text
    sequence before the decoder runs (``encoder_tokens[name]`` = placeholder id)."""

    def __init__(self, decoder: nn.Module, encoders: Dict[str, nn.Module], encoder_tokens: Dict[str, int], decoder_trainable: bool = False, encoders_trainable: Union[bool, Dict[str, bool]] = False, fusion_trainable: bool = True):
        super().__init__()
        if encoders.keys() != encoder_tokens.keys() or (not isinstance(encoders_trainable, bool) and encoders.keys() != encoders_trainable.keys()):
            raise ValueError(f"Found mismatched keys in encoders, encoder_tokens, and/or encoders_trainable. Expected {encoders.keys()}")
        self.decoder = decoder
        self.encoders = nn.ModuleDict(encoders)
        self.encoder_tokens = dict(encoder_tokens)
        self.encoders_trainable = {k: encoders_trainable for k in encoders} if isinstance(encoders_trainable, bool) else dict(encoders_trainable)
        trainable = set()
        for name, on in self.encoders_trainable.items():
            if on:
                trainable |= {f"encoders.{name}.{n}" for n, _ in self.encoders[name].named_parameters()}
        if decoder_trainable:
            trainable |= {f"decoder.{n}" for n, _ in decoder.named_parameters()}
        self._freeze_except(trainable, fusion_trainable)

    def forward(self, tokens: torch.Tensor, *, mask=None, encoder_input: Optional[Dict[str, Dict[str, Any]]] = None, input_pos: Optional[torch.Tensor] = None, **kwargs: Any) -> torch.Tensor:
        encoder_input = encoder_input or {}
        unknown = [k for k in encoder_input if k not in self.encoders]
        if unknown:
            raise ValueError(f"Found missing keys of encoder_input in instantiated encoders. Got {list(self.encoders.keys())}, expected {list(encoder_input.keys())}.")
        special = torch.tensor(list(self.encoder_tokens.values()), device=tokens.device)
        is_text = ~torch.isin(tokens, special)
        # placeholders are embedded with id 0 and then overwritten
        embeds = ops.embed_tokens(self.decoder.tok_embeddings, torch.where(is_text, tokens, torch.zeros_like(tokens)))
        for name, inp in encoder_input.items():
            enc = self.encoders[name](**inp).reshape(-1, embeds.shape[-1])
            slot = (tokens == self.encoder_tokens[name]).unsqueeze(-1)
            embeds = embeds.masked_scatter(slot, enc.to(embeds.dtype))
        return self.decoder(tokens=None, mask=mask, input_pos=input_pos, input_embeds=embeds)
