"""Rule-based rewards of the asynchronous GRPO recipe (parity: torchtune/dev/rl/rewards.py:20-316).

The reference delegates answer equivalence to the ``math_verify`` package; here :func:`answers_match` compares the last number
(integer, decimal, fraction, thousands separators, percent or currency signs stripped) of both strings, which is what GSM8K-style
answers need, and falls back to a whitespace-insensitive string comparison."""
from __future__ import annotations

import re
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from fractions import Fraction
from typing import Dict, List, Optional, Tuple

import torch

_NUMBER = re.compile(r"-?\d[\d,]*(?:\.\d+)?(?:\s*/\s*-?\d[\d,]*(?:\.\d+)?)?")


def _last_number(text: str) -> Optional[Fraction]:
    found = _NUMBER.findall(text.replace("$", "").replace("%", ""))
    if not found:
        return None
    raw = found[-1].replace(",", "").replace(" ", "")
    try:
        if "/" in raw:
            num, den = raw.split("/")
            return Fraction(num) / Fraction(den)
        return Fraction(raw)
    except (ValueError, ZeroDivisionError):
        return None


def answers_match(gold: str, attempt: str) -> bool:
    a, b = _last_number(gold), _last_number(attempt)
    if a is not None and b is not None:
        return a == b
    return "".join(gold.split()).lower() == "".join(attempt.split()).lower() and bool(gold.strip())


@dataclass
class RewardOutput:
    """Total reward ``[b]`` (what advantages are computed from), successes ``[b]`` and optional named parts for logging."""

    reward_base_name: str
    total_reward: torch.Tensor
    successes: torch.Tensor
    rewards: Optional[Dict[str, torch.Tensor]] = field(default_factory=dict)

    def log(self, prefix: str = "") -> Dict[str, float]:
        base = f"{prefix}/{self.reward_base_name}" if prefix else self.reward_base_name
        out = {f"{base}/{name}": r.float().mean().item() for name, r in (self.rewards or {}).items()}
        out[base] = self.total_reward.float().mean().item()
        out[f"{base}/successes"] = self.successes.float().mean().item()
        return out


class Reward(ABC):
    @abstractmethod
    def __call__(self, completion_ids: torch.Tensor, completions: List[str], answers: List[str]) -> RewardOutput:
        """``completion_ids`` ``[b, L]``, decoded ``completions`` and gold ``answers`` (one per completion) → :class:`RewardOutput`."""


class FormattedMathCorrectnessReward(Reward):
    """``positive_reward`` when the text inside ``<answer_tag>…</answer_tag>`` (the whole completion when the tag is missing) equals
    the gold answer, half of it when the gold answer merely appears in the completion, ``negative_reward`` otherwise."""

    def __init__(self, answer_tag: str, positive_reward: float, negative_reward: float = 0.0):
        self.answer_tag, self.positive_reward, self.negative_reward = answer_tag, positive_reward, negative_reward
        self._pattern = re.compile(rf"<{answer_tag}>(.*?)</{answer_tag}>", re.DOTALL)

    def __call__(self, completion_ids, completions, answers) -> RewardOutput:
        vals = []
        for completion, answer in zip(completions, answers):
            m = self._pattern.search(completion)
            attempt = m.group(1) if m else completion
            if answers_match(answer, attempt):
                vals.append(self.positive_reward)
            elif answer and answer in completion:
                vals.append(self.positive_reward / 2)
            else:
                vals.append(self.negative_reward)
        r = torch.tensor(vals, dtype=torch.float32)
        return RewardOutput("math_correctness", r, (r == self.positive_reward).float())


class ThinkingAnswerFormattingReward(Reward):
    """Soft format reward (exactly one think block followed by exactly one answer block) plus strict format reward (the
    completion is nothing but the two blocks, each on its own lines)."""

    def __init__(self, think_tag: str, answer_tag: str, positive_reward: float, negative_reward: float = 0.0):
        self.think_tag, self.answer_tag, self.positive_reward, self.negative_reward = think_tag, answer_tag, positive_reward, negative_reward

    def __call__(self, completion_ids, completions, answers) -> RewardOutput:
        t, a = self.think_tag, self.answer_tag
        think, answer = re.compile(rf"<{t}>.*?</{t}>", re.DOTALL), re.compile(rf"<{a}>.*?</{a}>", re.DOTALL)
        strict = re.compile(rf"^<{t}>\n.*?\n</{t}>\n<{a}>\n.*?\n</{a}>\n$", re.DOTALL | re.MULTILINE)
        soft_vals, strict_vals = [], []
        for c in completions:
            strict_vals.append(self.positive_reward if strict.match(c) else self.negative_reward)
            ts, as_ = think.findall(c), answer.findall(c)
            ok = len(ts) == 1 and len(as_) == 1 and c.find(ts[0]) < c.find(as_[0])
            soft_vals.append(self.positive_reward if ok else self.negative_reward)
        soft, hard = torch.tensor(soft_vals, dtype=torch.float32), torch.tensor(strict_vals, dtype=torch.float32)
        total = soft + hard
        return RewardOutput("formatting", total, (total >= self.positive_reward).float(), {"soft_format_reward": soft, "strict_format_reward": hard})


def extract_tags(text: str) -> Tuple[str, str]:
    """``(chain of thought, answer)`` bodies of the first ``<think>`` / ``<answer>`` blocks (empty when absent)."""
    think, answer = re.search(r"<think>(.*?)</think>", text, re.DOTALL), re.search(r"<answer>(.*?)</answer>", text, re.DOTALL)
    return (think.group(1).strip() if think else ""), (answer.group(1).strip() if answer else "")


def at_least_one_space_between_think_tags(cot: str, answer: str, potential_answer: str) -> Tuple[float, float]:
    return (1.0, 1.0) if len(cot) > 0 else (0.0, 0.0)


def math_response_correct(cot: str, answer: str, potential_answer: str) -> Tuple[float, float]:
    if potential_answer is None:
        return 0.0, 0.0
    if answers_match(answer, potential_answer):
        return 100.0, 1.0
    if answer in potential_answer:
        return 50.0, 0.0
    return (1.0, 0.0) if len(potential_answer) > 0 else (0.0, 0.0)


def batched_rewards(tokenizer, completions: torch.Tensor, answers: List[str], device: torch.device):
    """``completions`` ``[B, G, L]`` → ``(rewards [B, G, F], successes [B, G, F], {"func_names": [...]})`` for the two functional
    rewards above (the prompt already opened the think tag)."""
    funcs = [at_least_one_space_between_think_tags, math_response_correct]
    b, g, _ = completions.shape
    rewards, successes = torch.zeros(b, g, len(funcs), device=device), torch.zeros(b, g, len(funcs), device=device)
    for i in range(b):
        for j in range(g):
            cot, attempt = extract_tags("<think>" + tokenizer.decode(completions[i, j].tolist()))
            for f, fn in enumerate(funcs):
                r, s = fn(cot, answers[i], attempt)
                rewards[i, j, f] += r
                successes[i, j, f] += s
    return rewards, successes, {"func_names": [f.__name__ for f in funcs]}
