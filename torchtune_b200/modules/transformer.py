"""Decoder layers and the decoder stack (parity: torchtune/modules/transformer.py:17-689)."""
from __future__ import annotations

import copy
from typing import Callable, List, Optional, Union

import torch
from torch import nn

from .. import ops
from ..ops.mask import AttentionMask
from .attention import MaskLike, MultiHeadAttention


class TransformerSelfAttentionLayer(nn.Module):
    """Pre-norm block: ``h = x + sa_scale(attn(sa_norm(x)))``, ``out = h + mlp_scale(mlp(mlp_norm(h)))``.

    ``mask_mod(mask, bsz, seq_len)`` may rewrite the mask for this layer only (Llama-4
    local attention layers)."""

    def __init__(
        self,
        attn: MultiHeadAttention,
        mlp: nn.Module,
        *,
        sa_norm: Optional[nn.Module] = None,
        mlp_norm: Optional[nn.Module] = None,
        sa_scale: Optional[nn.Module] = None,
        mlp_scale: Optional[nn.Module] = None,
        mask_mod: Optional[Callable[[MaskLike, int, int], MaskLike]] = None,
    ) -> None:
        super().__init__()
        self.attn = attn
        self.mlp = mlp
        self.sa_norm = sa_norm or nn.Identity()
        self.mlp_norm = mlp_norm or nn.Identity()
        self.sa_scale = sa_scale or nn.Identity()
        self.mlp_scale = mlp_scale or nn.Identity()
        self.mask_mod = mask_mod

    def setup_caches(self, batch_size: int, dtype: torch.dtype, *, encoder_max_seq_len: int, decoder_max_seq_len: int) -> None:
        self.attn.setup_cache(batch_size, dtype, max_seq_len=decoder_max_seq_len)

    def caches_are_setup(self) -> bool:
        return self.attn.kv_cache is not None

    def caches_are_enabled(self) -> bool:
        return self.attn.cache_enabled

    def reset_cache(self) -> None:
        self.attn.reset_cache()

    @property
    def _fuse_residual_attn(self) -> bool:
        # exact types only: converted or derived modules (tensor-parallel attention, adapters on the whole block) keep the plain path
        return type(self.sa_scale) is nn.Identity and type(self.attn) is MultiHeadAttention

    @property
    def _fuse_residual_mlp(self) -> bool:
        from .feed_forward import FeedForward

        return type(self.mlp_scale) is nn.Identity and type(self.mlp) is FeedForward

    def forward(self, x: torch.Tensor, *, mask: MaskLike = None, input_pos: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        if self.mask_mod is not None:
            mask = self.mask_mod(mask, x.shape[0], x.shape[1])
        normed = self.sa_norm(x)
        # Without layer scales the two residual additions ride in the epilogues of the attention output projection and of the MLP down
        # projection (modules that take a ``residual`` argument); otherwise they are separate additions.
        if self._fuse_residual_attn:
            h = self.attn(normed, normed, mask=mask, input_pos=input_pos, residual=x)
        else:
            h = self.sa_scale(self.attn(normed, normed, mask=mask, input_pos=input_pos)) + x
        if self._fuse_residual_mlp:
            return self.mlp(self.mlp_norm(h), residual=h)
        return h + self.mlp_scale(self.mlp(self.mlp_norm(h)))


class TransformerCrossAttentionLayer(nn.Module):
    """Cross-attention block over encoder tokens.  Query rows whose encoder mask is
    empty contribute nothing (attention and MLP outputs are zeroed for them)."""

    def __init__(
        self,
        attn: MultiHeadAttention,
        mlp: nn.Module,
        *,
        ca_norm: Optional[nn.Module] = None,
        mlp_norm: Optional[nn.Module] = None,
        ca_scale: Optional[nn.Module] = None,
        mlp_scale: Optional[nn.Module] = None,
    ) -> None:
        super().__init__()
        if attn.pos_embeddings is not None:
            raise AssertionError("Doesn't support positional embeddings for cross attention, because q and k are different sequences.")
        self.attn = attn
        self.mlp = mlp
        self.ca_norm = ca_norm or nn.Identity()
        self.mlp_norm = mlp_norm or nn.Identity()
        self.ca_scale = ca_scale or nn.Identity()
        self.mlp_scale = mlp_scale or nn.Identity()

    def setup_caches(self, batch_size: int, dtype: torch.dtype, *, encoder_max_seq_len: int, decoder_max_seq_len: int) -> None:
        self.attn.setup_cache(batch_size, dtype, encoder_max_seq_len)

    def caches_are_setup(self) -> bool:
        return self.attn.kv_cache is not None

    def caches_are_enabled(self) -> bool:
        return self.attn.cache_enabled

    def reset_cache(self) -> None:
        self.attn.reset_cache()

    @staticmethod
    def _skip_mask(mask: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """``[b, s_q, 1]`` True where a query row may attend to nothing; such rows are
        un-masked inside attention (avoids NaN) and zeroed afterwards."""
        if mask is None:
            return None
        if mask.dtype == torch.bool:
            m = ~mask
        else:
            m = torch.isneginf(mask)
        return torch.all(m, dim=-1, keepdim=True)

    def forward(
        self,
        x: torch.Tensor,
        *,
        encoder_input: Optional[torch.Tensor] = None,
        encoder_mask: Optional[torch.Tensor] = None,
        **kwargs,
    ) -> torch.Tensor:
        empty_cache = not self.caches_are_enabled() or self.attn.kv_cache.size == 0
        if encoder_input is None and empty_cache:
            return x
        skip = self._skip_mask(encoder_mask)
        if encoder_mask is not None:
            encoder_mask = encoder_mask.masked_fill(skip, True)
        attn_out = self.attn(self.ca_norm(x), encoder_input, mask=encoder_mask)
        if skip is not None:
            attn_out = attn_out.masked_fill(skip, 0)
        h = self.ca_scale(attn_out) + x
        mlp_out = self.mlp(self.mlp_norm(h))
        if skip is not None:
            mlp_out = mlp_out.masked_fill(skip, 0)
        return h + self.mlp_scale(mlp_out)


def _get_clones(module: nn.Module, n: int) -> nn.ModuleList:
    return nn.ModuleList([copy.deepcopy(module) for _ in range(n)])


class TransformerDecoder(nn.Module):
    """``tok_embeddings → layers → norm → output``.

    * ``skip_output_layer=True`` returns the normalised hidden states so a fused
      linear+loss operator can apply ``output`` itself.
    * ``num_output_chunks > 0`` returns the logits as a list of sequence chunks.
    * Materialised logits are fp32.
    """

    def __init__(
        self,
        *,
        tok_embeddings: nn.Embedding,
        layers: Union[nn.Module, List[nn.Module], nn.ModuleList],
        max_seq_len: int,
        num_heads: int,
        head_dim: int,
        norm: nn.Module,
        output: Union[nn.Linear, Callable],
        num_layers: Optional[int] = None,
        output_hidden_states: Optional[List[int]] = None,
    ) -> None:
        super().__init__()
        if isinstance(layers, nn.ModuleList):
            pass
        elif isinstance(layers, list):
            layers = nn.ModuleList(layers)
        else:
            if not isinstance(layers, nn.Module):
                raise AssertionError("num_layers is defined, layers must be a module")
            if num_layers is None:
                raise AssertionError("num_layers must be defined if layers is not a list")
            layers = _get_clones(layers, num_layers)
        self.tok_embeddings = tok_embeddings
        self.layers = layers
        self.norm = norm
        self.output = output
        self.output_hidden_states = output_hidden_states or []
        self.max_seq_len = max_seq_len
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.causal_mask = None
        self.num_output_chunks = 0
        self.skip_output_layer = False
        # cap·tanh(logits/cap) applied to the logits (Gemma-2); 0 = none.  A loss that takes the hidden states instead
        # (``skip_output_layer``) reads this attribute and applies the cap itself.
        self.logit_softcap = 0.0
        self.encoder_max_cache_seq_len = None
        self.decoder_max_cache_seq_len = None

    # -- output chunking (deprecated path kept for API parity) -------------
    def set_num_output_chunks(self, num_output_chunks: int) -> None:
        self.num_output_chunks = num_output_chunks

    # -- KV caches -----------------------------------------------------------
    def setup_caches(
        self,
        batch_size: int,
        dtype: torch.dtype,
        *,
        encoder_max_seq_len: Optional[int] = None,
        decoder_max_seq_len: Optional[int] = None,
    ) -> None:
        kinds = [getattr(m, "inner_cls", type(m)) for m in self.modules()]  # sees through checkpoint wrappers
        has_enc = any(issubclass(k, TransformerCrossAttentionLayer) for k in kinds)
        has_dec = any(issubclass(k, TransformerSelfAttentionLayer) for k in kinds)
        if has_enc:
            self.encoder_max_cache_seq_len = encoder_max_seq_len if encoder_max_seq_len is not None else self.max_seq_len
        if has_dec:
            self.decoder_max_cache_seq_len = decoder_max_seq_len if decoder_max_seq_len is not None else self.max_seq_len
        for layer in self.layers:
            layer.setup_caches(
                batch_size,
                dtype,
                encoder_max_seq_len=self.encoder_max_cache_seq_len,
                decoder_max_seq_len=self.decoder_max_cache_seq_len,
            )

    def caches_are_setup(self) -> bool:
        return self.layers[0].caches_are_setup()

    def caches_are_enabled(self) -> bool:
        return self.layers[0].caches_are_enabled()

    def reset_caches(self) -> None:
        if not self.caches_are_enabled():
            raise RuntimeError("Key value caches are not setup. Call model.setup_caches first.")
        for layer in self.layers:
            layer.reset_cache()

    # -- forward ---------------------------------------------------------------
    def _cap(self, logits: torch.Tensor) -> torch.Tensor:
        cap = float(self.logit_softcap)
        return logits if cap <= 0.0 else torch.tanh(logits / cap) * cap

    def chunked_output(self, last_hidden_state: torch.Tensor) -> List[torch.Tensor]:
        return [self._cap(self.output(chunk)) for chunk in last_hidden_state.tensor_split(self.num_output_chunks, dim=1)]

    def _validate_inputs(self, seq_len, mask=None, encoder_input=None, encoder_mask=None, input_pos=None) -> None:
        if seq_len > self.max_seq_len:
            raise ValueError(f"seq_len ({seq_len}) of input tensor should be smaller than max_seq_len ({self.max_seq_len})")
        if self.caches_are_enabled():
            if mask is None:
                raise ValueError("KV-caches for self-attention layers are setup for inference mode, causal masks must be provided! Use the `mask` arg to provide a causal mask.")
            if encoder_input is not None and encoder_mask is None:
                raise ValueError("KV-caches for cross-attention/fusion layers are setup for inference mode and you seem to be using encoder_input, causal masks must be provided! Use the `encoder_mask` arg to provide a causal mask.")
            if input_pos is None:
                raise ValueError("KV-caches are setup for inference mode, input positions must be provided!")

    def forward(
        self,
        tokens: Optional[torch.Tensor] = None,
        *,
        mask: MaskLike = None,
        encoder_input: Optional[torch.Tensor] = None,
        encoder_mask: Optional[torch.Tensor] = None,
        input_pos: Optional[torch.Tensor] = None,
        input_embeds: Optional[torch.Tensor] = None,
    ) -> Union[torch.Tensor, List[torch.Tensor]]:
        if (tokens is None) == (input_embeds is None):
            raise ValueError("Exactly one of `tokens` or `input_embeds` must be provided.")
        seq_len = tokens.shape[1] if input_embeds is None else input_embeds.shape[1]
        self._validate_inputs(seq_len, mask=mask, encoder_input=encoder_input, encoder_mask=encoder_mask, input_pos=input_pos)
        h = ops.embed_tokens(self.tok_embeddings, tokens) if input_embeds is None else input_embeds
        hidden = []
        for i, layer in enumerate(self.layers):
            if i in self.output_hidden_states:
                hidden.append(h)
            h = layer(h, mask=mask, encoder_input=encoder_input, encoder_mask=encoder_mask, input_pos=input_pos)
        if len(self.layers) in self.output_hidden_states:
            hidden.append(h)
        h = self.norm(h)
        if self.skip_output_layer:
            output = h
        elif self.num_output_chunks > 0:
            output = self.chunked_output(h)
        else:
            output = self.unembed_normed(h)
        return output if not hidden else [*hidden, output]

    def unembed_normed(self, h: torch.Tensor) -> torch.Tensor:
        return self._cap(self.output(h).float())

    def unembed(self, h: torch.Tensor) -> torch.Tensor:
        """Final norm + output projection of a hidden state (fp32 logits)."""
        h = self.norm(h)
        if self.num_output_chunks > 0:
            return self.chunked_output(h)
        return self._cap(self.output(h).float())
