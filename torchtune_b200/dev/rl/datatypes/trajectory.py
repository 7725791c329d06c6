"""One prompt group on its way from the inference workers to the trainer (parity: torchtune/dev/rl/datatypes/trajectory.py:12-23).
The reference uses a ``tensordict.TensorClass``; a dataclass with the same fields plus ``to`` / ``stack`` is all the roles need."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, List, Optional

import torch


@dataclass
class Trajectory:
    query_responses: torch.Tensor  # [G, P + L] prompt (left-padded) followed by the sampled response (right-padded)
    responses: torch.Tensor  # [G, L]
    logprobs: torch.Tensor  # [G, L] under the policy that sampled them
    ref_logprobs: Optional[torch.Tensor]  # [G, L] under the frozen reference policy (filled by post-processing)
    query_response_padding_masks: torch.Tensor  # [G, P + L] True = real token
    seq_lens: torch.Tensor  # [G] response lengths
    answers: List[str]
    policy_version: int
    advantages: Optional[torch.Tensor] = None  # [G]
    reward_outputs: List[Any] = field(default_factory=list)
    sequence_ids: List[str] = field(default_factory=list)

    def to(self, device) -> "Trajectory":
        return Trajectory(**{f.name: (getattr(self, f.name).to(device) if torch.is_tensor(getattr(self, f.name)) else getattr(self, f.name)) for f in fields(self)})

    @staticmethod
    def stack(items: List["Trajectory"], pad_id: int = 0) -> "Trajectory":
        """Concatenate groups along the batch dimension (sequence dimensions are right-padded to the longest)."""

        def cat(name: str, fill):
            ts = [getattr(t, name) for t in items]
            if ts[0] is None:
                return None
            if ts[0].dim() == 1:
                return torch.cat(ts)
            width = max(t.shape[1] for t in ts)
            return torch.cat([torch.nn.functional.pad(t, (0, width - t.shape[1]), value=fill) for t in ts])

        return Trajectory(
            query_responses=cat("query_responses", pad_id), responses=cat("responses", pad_id), logprobs=cat("logprobs", 0.0), ref_logprobs=cat("ref_logprobs", 0.0),
            query_response_padding_masks=cat("query_response_padding_masks", False), seq_lens=cat("seq_lens", 0), answers=[a for t in items for a in t.answers],
            policy_version=min(t.policy_version for t in items), advantages=cat("advantages", 0.0), reward_outputs=[r for t in items for r in t.reward_outputs],
            sequence_ids=[s for t in items for s in t.sequence_ids],
        )
