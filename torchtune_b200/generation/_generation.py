"""Batched autoregressive sampling (parity: torchtune/generation/_generation.py:14-443)."""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

from ..modules import TransformerDecoder


def multinomial_sample_one(probs: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """Exponential-race sampling: ``argmax(p / q)`` with ``q ~ Exp(1)`` draws from ``p``."""
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(dtype=torch.int)


def _exponential_like(shape, device, rng: Optional[torch.Generator] = None) -> torch.Tensor:
    u = torch.rand(shape, generator=rng, device=device)
    eps = torch.finfo(u.dtype).eps / 2
    return -torch.log(torch.clamp(1.0 - u, min=eps))  # avoids log(0)


def sample(logits: torch.Tensor, *, temperature: float = 1.0, top_k: Optional[int] = None, q: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Temperature + optional top-k, then one draw per row; returns ``[..., 1]`` int tokens."""
    if logits.is_cuda:
        from .. import ops

        qq = q if q is not None else _exponential_like(logits.shape, logits.device)
        tokens = ops.sample_tokens(logits, qq.float() if qq.dtype != torch.float32 else qq, temperature, top_k)
        if tokens is not None:
            return tokens
        q = qq
    logits = logits / max(temperature, 1e-5)
    if top_k is not None:
        kth = torch.topk(logits, min(top_k, logits.size(-1))).values[..., -1:]
        logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
    probs = torch.softmax(logits, dim=-1)
    if q is None:
        q = _exponential_like(probs.shape, probs.device)
    return multinomial_sample_one(probs, q)


def generate_next_token(model: TransformerDecoder, input_pos: torch.Tensor, x: torch.Tensor, q: Optional[torch.Tensor] = None, *, mask: Optional[torch.Tensor] = None, temperature: float = 1.0, top_k: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One forward pass; samples from the last position.  Returns ``(tokens [b,1], logits [b,1,v])``."""
    logits = model(x, input_pos=input_pos, mask=mask)[:, -1]
    return sample(logits.clone(), temperature=temperature, top_k=top_k, q=q), logits.unsqueeze(1)


def update_stop_tokens_tracker(tokens: torch.Tensor, stop_tokens: torch.Tensor, stop_token_reached: torch.Tensor) -> torch.Tensor:
    stop_token_reached |= torch.isin(tokens, stop_tokens).flatten()
    return stop_token_reached


def get_causal_mask_from_padding_mask(padding_mask: torch.Tensor, target_seq_len: Optional[int] = None) -> torch.Tensor:
    """``padding_mask`` ``[b, s]`` (True = real token) → boolean ``[b, s, target]`` causal mask
    that also hides padding keys; every position can attend to itself."""
    bsz, seq_len = padding_mask.shape
    target = seq_len if target_seq_len is None else target_seq_len
    if target < seq_len:
        raise AssertionError("target_seq_len cannot be shorter than the sequence length of the padding mask.")
    causal = torch.tril(torch.ones(seq_len, target, dtype=torch.bool, device=padding_mask.device)).repeat(bsz, 1, 1)
    causal[:, :, :seq_len] &= padding_mask[:, None, :]
    idx = torch.arange(seq_len, device=padding_mask.device)
    causal[:, idx, idx] = True
    return causal


def get_position_ids_from_padding_mask(padding_mask: torch.Tensor) -> torch.Tensor:
    """Positions that start counting at the first real token of each (left-padded) row."""
    return ((padding_mask.cumsum(-1) - 1) * padding_mask).to(torch.int)


@torch.no_grad()
def generate(
    model: TransformerDecoder,
    prompt: torch.Tensor,
    *,
    max_generated_tokens: int,
    pad_id: int = 0,
    temperature: float = 1.0,
    top_k: Optional[int] = None,
    stop_tokens: Optional[List[int]] = None,
    rng: Optional[torch.Generator] = None,
    custom_generate_next_token: Optional[Callable] = None,
    return_logits: bool = True,
    stop_group=None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Sample up to ``max_generated_tokens`` continuations of ``prompt`` (``[b, s]`` or ``[s]``,
    left-padded with ``pad_id`` when lengths differ).  With KV caches enabled on the model each
    step feeds only the new token.  Returns ``(tokens [b, s + n], logits [b, n, vocab])``;
    tokens after a stop token are replaced by ``pad_id`` and their logits zeroed.

    ``return_logits=False`` keeps no per-step logits (the second result is ``None``), which is what a rollout needs when the
    log-probabilities are recomputed afterwards.  ``stop_group`` is a process group (``True`` for the default one): the loop then
    ends only when every rank of the group has seen a stop token in every row, so ranks that hold shards of one model keep
    issuing the same number of forward passes (parity: torchtune/dev/rl/generation.py:29-190)."""
    prompt = prompt.view(1, -1) if prompt.ndim == 1 else prompt
    bsz, prompt_len = prompt.shape
    total_len = prompt_len + max_generated_tokens
    device = prompt.device
    incremental = model.caches_are_enabled()
    mask_width = model.decoder_max_cache_seq_len if incremental else total_len

    real = prompt != pad_id
    if not real.all():
        real = torch.nn.functional.pad(real, (0, max_generated_tokens), value=True)
        masks = get_causal_mask_from_padding_mask(real, target_seq_len=mask_width)
        input_pos = get_position_ids_from_padding_mask(real)
    else:
        masks = torch.tril(torch.ones(total_len, mask_width, dtype=torch.bool, device=device)).unsqueeze(0)
        input_pos = torch.arange(total_len, device=device).unsqueeze(0)

    def draw_q():
        return None if rng is None else _exponential_like((bsz, model.tok_embeddings.num_embeddings), device, rng)

    first_mask = masks[:, :prompt_len] if incremental else masks[:, :prompt_len, :prompt_len]
    tokens, logits = generate_next_token(model, input_pos=input_pos[:, :prompt_len].squeeze(), mask=first_mask, x=prompt, temperature=temperature, top_k=top_k, q=draw_q())
    out_tokens = torch.cat([prompt, tokens], dim=-1)
    logit_steps = [logits] if return_logits else None  # joined once at the end: joining every step copies the whole history each time
    pos = prompt_len

    def everyone_done(flags: torch.Tensor) -> bool:
        done = flags.all()
        if stop_group is not None and torch.distributed.is_available() and torch.distributed.is_initialized():
            done = done.to(torch.int32)
            torch.distributed.all_reduce(done, op=torch.distributed.ReduceOp.MIN, group=None if stop_group is True else stop_group)
        return bool(done)

    stop = torch.tensor(stop_tokens, device=device, dtype=tokens.dtype) if stop_tokens else None
    reached = torch.zeros(bsz, dtype=torch.bool, device=device)
    keep = torch.ones(bsz, prompt_len + 1, dtype=torch.int32, device=device)
    if stop is not None:
        reached = update_stop_tokens_tracker(tokens, stop, reached)
        if everyone_done(reached):
            return out_tokens, (logits if return_logits else None)

    step_fn = custom_generate_next_token or generate_next_token
    for _ in range(max_generated_tokens - 1):
        if stop is not None:
            keep = torch.cat([keep, (~reached).reshape(bsz, 1).to(torch.int32)], dim=-1)
        if incremental:
            cur_pos, cur_mask, x = input_pos[:, pos].contiguous(), masks[:, pos, None, :].contiguous(), tokens.clone()
        else:
            cur_pos, cur_mask, x = input_pos[:, : pos + 1], masks[:, : pos + 1, : pos + 1], out_tokens.clone()
        tokens, logits = step_fn(model, input_pos=cur_pos, x=x, mask=cur_mask, temperature=temperature, top_k=top_k, q=draw_q())
        out_tokens = torch.cat([out_tokens, tokens], dim=-1)
        if return_logits:
            logit_steps.append(logits)
        pos += 1
        if stop is not None:
            reached = update_stop_tokens_tracker(tokens, stop, reached)
            if everyone_done(reached):
                break

    all_logits = torch.cat(logit_steps, dim=1) if return_logits else None
    if stop is not None:
        out_tokens = out_tokens * keep + pad_id * (1 - keep) if keep.shape == out_tokens.shape else out_tokens
        if return_logits:
            all_logits = all_logits * keep[:, -all_logits.shape[1] :, None]
    return out_tokens, all_logits
