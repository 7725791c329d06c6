"""Prompt datasets for RL fine-tuning (parity: torchtune/dev/grpo/data.py:25-105, gsm8k.py:25-140)."""
from __future__ import annotations

import re
from typing import Any, Callable, Dict, List, Mapping, Optional, TypedDict, Union

import torch
from torch.nn.utils.rnn import pad_sequence
from torch.utils.data import Dataset

from ...data import CROSS_ENTROPY_IGNORE_IDX
from ...datasets._sft import SFTDataset, _load

BASE_PROMPT = (
    "A conversation between User and Assistant. The user asks a question, and the Assistant solves it. "
    "The assistant first thinks about the reasoning process in the mind and then provides the user with the answer. "
    "The reasoning process and answer are enclosed within <think></think> and <answer></answer> tags, respectively, "
    "i.e., <think>reasoning process here</think> <answer>answer here</answer>. User: %s. Assistant: <think>"
)


class ReasoningProblem(TypedDict):
    """What a ``problem_transform`` returns: the question, the worked solution and the final answer."""

    question: str
    cot: str
    answer: str


class RLDataset(Dataset):
    """Rows → ``{"question", "tokens", "mask", "answer"}``; ``problem_transform`` maps a raw row to ``question`` / ``answer``."""

    def __init__(self, *, source: str, problem_transform: Callable, tokenizer: Any, filter_fn: Optional[Callable] = None, filter_kwargs: Optional[Dict[str, Any]] = None, **load_dataset_kwargs: Any) -> None:
        self._problem_transform, self._tokenizer = problem_transform, tokenizer
        self._data = _load(source, **load_dataset_kwargs)
        if filter_fn is not None:
            self._data = self._data.filter(filter_fn, **(filter_kwargs or {}))

    def __len__(self) -> int:
        return len(self._data)

    def __getitem__(self, index: int) -> Dict[str, Any]:
        problem = self._problem_transform(self._data[index])
        question = BASE_PROMPT % problem["question"]
        tokens = self._tokenizer.encode(question, add_eos=False)
        return {"question": question, "tokens": tokens, "mask": [1] * len(tokens), "answer": problem["answer"]}


def padded_collate_rl(batch: List[Dict[str, Any]], padding_idx: int = 0, ignore_idx: int = CROSS_ENTROPY_IGNORE_IDX) -> Dict[str, Union[torch.Tensor, List[str]]]:
    tokens = pad_sequence([torch.tensor(x["tokens"]) for x in batch], batch_first=True, padding_value=padding_idx)
    return {"tokens": tokens.long(), "answers": [x["answer"] for x in batch], "text": [x["question"] for x in batch]}


def normalize_gsm(problem: Mapping[str, str]) -> ReasoningProblem:
    """GSM8K rows end with ``#### <answer>``; the text before it is the worked solution."""
    cot, _, answer = problem["answer"].partition("#### ")
    return {"question": problem["question"], "cot": cot.strip(), "answer": answer.strip()}


def sft_gsm_transform(problem: Mapping[str, str]) -> Dict[str, str]:
    """Supervised target in the tag format the RL prompt asks for (calculator annotations ``<<…>>`` removed)."""
    p = normalize_gsm(problem)
    cot = re.sub(r"<<.*?>>", "", p["cot"])
    return {"input": BASE_PROMPT % p["question"], "output": f"{cot}</think> <answer>{p['answer']}</answer>"}


def gsm8k_dataset(tokenizer: Any, *, source: str = "openai/gsm8k", filter_fn: Optional[Callable] = None, split: str = "train", name: str = "main", partition: Optional[str] = None, **load_dataset_kwargs: Any) -> RLDataset:
    """GSM8K as an RL prompt dataset; ``partition="a-b/n"`` keeps rows whose index modulo ``n`` lies in ``[a, b]``."""

    def _keep(_row, idx, lo=0, hi=0, n=1):
        return lo <= idx % n <= hi

    kwargs: Dict[str, Any] = {}
    if partition is not None:
        span, n = partition.split("/")
        lo, hi = span.split("-")
        filter_fn = lambda row, idx: _keep(row, idx, int(lo), int(hi), int(n))  # noqa: E731
        kwargs["filter_kwargs"] = {"with_indices": True}
    return RLDataset(source=source, name=name, tokenizer=tokenizer, problem_transform=normalize_gsm, filter_fn=filter_fn, split=split, **kwargs, **load_dataset_kwargs)


def gsm8k_sft(tokenizer: Any, *, source: str = "openai/gsm8k", filter_fn: Optional[Callable] = None, split: str = "train", name: str = "main", partition: Optional[str] = None, **load_dataset_kwargs: Any) -> SFTDataset:
    """GSM8K as a supervised dataset in the RL answer format (warm-up before GRPO)."""
    from ...data import InputOutputToMessages

    class _Rows:
        def __call__(self, row):
            return InputOutputToMessages()(sft_gsm_transform(row))

    return SFTDataset(source=source, message_transform=_Rows(), model_transform=tokenizer, filter_fn=filter_fn, split=split, name=name, **load_dataset_kwargs)


def reasoning_dataset(tokenizer: Any, *, source: str, question_column: str = "question", answer_column: str = "answer", filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> RLDataset:
    """Any dataset with a question and a final-answer column (local ``json`` / ``csv`` files or a hub dataset)."""

    def _transform(row: Mapping[str, Any]) -> Dict[str, str]:
        return {"question": str(row[question_column]), "cot": "", "answer": str(row[answer_column])}

    return RLDataset(source=source, tokenizer=tokenizer, problem_transform=_transform, filter_fn=filter_fn, split=split, **load_dataset_kwargs)
