"""Sequence-level helpers: truncation at stop tokens and log-probability reductions
(parity: torchtune/rlhf/sequence_processing.py:13-193)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

from ..data._common import CROSS_ENTROPY_IGNORE_IDX


def truncate_sequence_at_first_stop_token(sequences: torch.Tensor, stop_tokens: torch.Tensor, fill_value: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Everything *after* the first stop token of each row is replaced by ``fill_value``
    (in place).  Returns ``(padding_mask, sequences)`` with the mask True on replaced slots."""
    is_stop = torch.isin(sequences, stop_tokens)
    seen = torch.cumsum(is_stop, dim=1)
    padding_mask = (seen > 1) | ((seen == 1) & ~is_stop)
    sequences[padding_mask] = fill_value
    return padding_mask, sequences


def logits_to_logprobs(logits: torch.Tensor, sequences: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """``log_softmax(logits / T)`` gathered at ``sequences`` → ``[b, s]`` (bf16 CUDA logits: fused kernel, fp32 result)."""
    from .. import ops

    fused = ops.logits_logprobs(logits, sequences, temperature)
    if fused is not None:
        return fused
    return torch.gather(F.log_softmax(logits / temperature, dim=-1), 2, sequences.unsqueeze(-1)).squeeze(-1)


def batched_logits_to_logprobs(logits: torch.Tensor, sequences: torch.Tensor, temperature: float = 1.0, chunk_size: int = 1) -> torch.Tensor:
    """Same as :func:`logits_to_logprobs`, processed ``chunk_size`` rows at a time to bound memory."""
    out = torch.empty(sequences.shape, dtype=torch.float32, device=logits.device)
    for lo in range(0, logits.shape[0], chunk_size):
        out[lo : lo + chunk_size] = logits_to_logprobs(logits[lo : lo + chunk_size].float(), sequences[lo : lo + chunk_size], temperature)
    return out


def get_batch_log_probs(logits: torch.Tensor, labels: torch.Tensor, label_pad_token_id: int = CROSS_ENTROPY_IGNORE_IDX, return_average_logprobs: bool = False) -> torch.Tensor:
    """Sum (or mean) over the sequence of ``log p(label_t | prefix)``: labels are shifted left by
    one against the logits and positions equal to ``label_pad_token_id`` are excluded."""
    if logits.shape[:-1] != labels.shape:
        raise ValueError("Logits (batch and sequence length dim) and labels must have the same shape.")
    labels = labels[:, 1:].clone()
    logits = logits[:, :-1, :]
    valid = labels != label_pad_token_id
    labels[~valid] = 0
    per_token = logits_to_logprobs(logits, labels, temperature=1.0)
    total = (per_token * valid).sum(-1)
    return total / valid.sum(-1) if return_average_logprobs else total


def truncate_sequence_for_logprobs(query_response_logits: torch.Tensor, context_length: int) -> torch.Tensor:
    """Logits that *predict* the response tokens of a (query, response) sequence."""
    return query_response_logits[:, context_length - 1 : -1]
