"""Vocabulary resizing (parity: torchtune/modules/embedding_utils.py:25-143)."""
from __future__ import annotations

import torch
from torch import nn

from .tied_linear import TiedLinear


def _need_to_resize(model: nn.Module, num_embeddings: int) -> bool:
    for attr in ("tok_embeddings", "output"):
        if not hasattr(model, attr):
            raise AttributeError(f"Model does not have a `{attr}` attribute; cannot resize token embeddings.")
    if not isinstance(model.tok_embeddings, nn.Embedding):
        raise AttributeError("`model.tok_embeddings` must be an nn.Embedding to be resized.")
    return model.tok_embeddings.num_embeddings != num_embeddings


@torch.no_grad()
def resize_token_embeddings(model: nn.Module, num_embeddings: int) -> None:
    """Grow or shrink ``tok_embeddings`` and ``output`` to ``num_embeddings`` rows; new rows
    are initialised to the mean of the existing rows.  Sharded models must be resized
    before sharding (the sharder owns flat buffers)."""
    if not _need_to_resize(model, num_embeddings):
        return
    old = model.tok_embeddings
    keep = min(old.num_embeddings, num_embeddings)
    new_emb = nn.Embedding(num_embeddings, old.embedding_dim, device=old.weight.device, dtype=old.weight.dtype)
    new_emb.weight[:keep] = old.weight[:keep]
    if num_embeddings > keep:
        new_emb.weight[keep:] = old.weight.float().mean(0, keepdim=True).to(old.weight.dtype)
    new_emb.weight.requires_grad_(old.weight.requires_grad)
    model.tok_embeddings = new_emb
    if isinstance(model.output, TiedLinear):
        model.output = TiedLinear(new_emb)
        return
    out = model.output
    new_out = type(out)(out.in_features, num_embeddings, bias=out.bias is not None, device=out.weight.device, dtype=out.weight.dtype)
    new_out.weight[:keep] = out.weight[:keep]
    if num_embeddings > keep:
        new_out.weight[keep:] = out.weight.float().mean(0, keepdim=True).to(out.weight.dtype)
    if out.bias is not None:
        new_out.bias[:keep] = out.bias[:keep]
        if num_embeddings > keep:
            new_out.bias[keep:] = out.bias.float().mean().to(out.bias.dtype)
    new_out.weight.requires_grad_(out.weight.requires_grad)
    model.output = new_out
