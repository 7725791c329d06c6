"""Rollout generation for reinforcement learning (parity: torchtune/dev/rl/generation.py:29-190, torchtune/dev/grpo/generation.py).

Same sampler as :func:`torchtune_b200.generation.generate` with the two behaviours a rollout wants: the per-step logits are
optional, and in a multi-process job the stop-token exit is agreed between ranks, so that ranks holding shards of one model never
disagree on the number of decoding steps."""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

from ... import generation as _generation


@torch.no_grad()
def generate(model, prompt: torch.Tensor, *, max_generated_tokens: int, pad_id: int = 0, temperature: float = 1.0, top_k: Optional[int] = None,
             stop_tokens: Optional[List[int]] = None, rng: Optional[torch.Generator] = None, custom_generate_next_token: Optional[Callable] = None,
             return_logits: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    return _generation.generate(model, prompt, max_generated_tokens=max_generated_tokens, pad_id=pad_id, temperature=temperature, top_k=top_k,
                                stop_tokens=stop_tokens, rng=rng, custom_generate_next_token=custom_generate_next_token, return_logits=return_logits,
                                stop_group=True)
