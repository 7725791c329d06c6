"""What an inference worker returns for one prompt (parity: torchtune/dev/rl/datatypes/request_output.py:16-88,
vllm_completion_output.py): the prompt's tokens and ``group_size`` sampled completions with their per-token log-probabilities."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import torch


@dataclass
class CompletionOutput:
    index: int
    token_ids: List[int]
    logprobs: List[float]  # log p(token) under the sampling policy, one per generated token
    finish_reason: str = "length"  # "stop" when a stop token ended the completion


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput] = field(default_factory=list)
    answer: str = ""
    policy_version: int = 0

    def padded(self, max_len: int, pad_id: int):
        """``(responses [G, max_len], logprobs [G, max_len], padding mask [G, max_len] True = padding)``."""
        g = len(self.outputs)
        tokens = torch.full((g, max_len), pad_id, dtype=torch.long)
        logprobs = torch.zeros(g, max_len)
        pad = torch.ones(g, max_len, dtype=torch.bool)
        for i, o in enumerate(self.outputs):
            n = min(len(o.token_ids), max_len)
            tokens[i, :n] = torch.tensor(o.token_ids[:n], dtype=torch.long)
            logprobs[i, :n] = torch.tensor(o.logprobs[:n])
            pad[i, :n] = False
        return tokens, logprobs, pad
