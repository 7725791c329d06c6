"""Rule-based rewards for reasoning completions (parity: torchtune/dev/grpo/rewards.py:14-110)."""
from __future__ import annotations

import re
from typing import Any, Dict, List, Tuple

import torch

_THINK = re.compile(r"<think>(.*?)</think>", re.DOTALL)
_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.DOTALL)


def extract_tags(text: str) -> Dict[str, List[str]]:
    """First ``<think>…</think>`` and ``<answer>…</answer>`` bodies (empty strings when absent)."""
    think, answer = _THINK.search(text), _ANSWER.search(text)
    return {"think": [think.group(1).strip() if think else ""], "answer": [answer.group(1).strip() if answer else ""]}


def shaped_correctness_reward(answer: str, completion: str) -> Tuple[float, float]:
    """Partial credit for format (one think tag +5, one answer tag +5), for the answer appearing (+10 contained, +20 exact)
    and 100 (success = 1) when the last answer tag is exactly right.  The prompt already opened ``<think>``."""
    tags = extract_tags("<think>" + completion.replace("<<", "").replace(">>", ""))
    reward, success = 0.0, 0.0
    if len(tags["answer"]) == 1:
        reward += 5.0
    if len(tags["think"]) == 1:
        reward += 5.0
    if any(a == answer for a in tags["answer"]):
        reward += 20.0
    if any(answer in a for a in tags["answer"]):
        reward += 10.0
    if tags["answer"] and tags["answer"][-1] == answer:
        reward, success = 100.0, 1.0
    return reward, success


def batch_shaped_correctness_reward(tokenizer: Any, completions: torch.Tensor, answers: List[str]) -> Tuple[torch.Tensor, torch.Tensor]:
    """``completions``: ``[B, G, L]`` token ids; returns rewards and successes ``[B, G]``."""
    b, g, _ = completions.shape
    rewards, successes = torch.zeros(b, g), torch.zeros(b, g)
    for i in range(b):
        for j in range(g):
            rewards[i, j], successes[i, j] = shaped_correctness_reward(answers[i], tokenizer.decode(completions[i, j].tolist()))
    return rewards, successes
