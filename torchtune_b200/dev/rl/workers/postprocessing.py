"""Reference-policy log-probabilities, rewards and group-relative advantages (parity:
torchtune/dev/rl/workers/postprocessing.py:29-312)."""
from __future__ import annotations

import queue
from typing import Any, List, Optional

import torch
from torch import nn

from .... import generation, rlhf
from ..datatypes import Trajectory
from ..rewards import Reward
from .replay import ReplayBuffer


class PostProcessingWorker:
    def __init__(self, *, ref_model: nn.Module, tokenizer, reward_functions: List[Reward], rollout_queue, replay_buffer: ReplayBuffer, device: torch.device,
                 temperature: float = 1.0, metric_logger=None, worker_id: int = 0):
        self.ref_model = ref_model.eval()
        for p in self.ref_model.parameters():
            p.requires_grad_(False)
        self.tokenizer, self.reward_functions, self.rollout_queue, self.replay_buffer = tokenizer, list(reward_functions), rollout_queue, replay_buffer
        self.device, self.temperature, self.metric_logger, self.worker_id = device, temperature, metric_logger, worker_id
        self.pad_id = getattr(tokenizer, "pad_id", 0)
        self.groups_done = 0

    @torch.no_grad()
    def process(self, traj: Trajectory) -> Trajectory:
        t = traj.to(self.device)
        ctx = t.query_responses.shape[1] - t.responses.shape[1]
        masks = generation.get_causal_mask_from_padding_mask(t.query_response_padding_masks)
        position_ids = generation.get_position_ids_from_padding_mask(t.query_response_padding_masks)
        logits = self.ref_model(t.query_responses, input_pos=position_ids, mask=masks)
        logits = rlhf.truncate_sequence_for_logprobs(logits, ctx)
        ref_logprobs = rlhf.logits_to_logprobs(logits, t.responses, self.temperature)
        pad = ~t.query_response_padding_masks[:, ctx:]
        ref_logprobs = ref_logprobs.masked_fill(pad, 0.0)
        completions = [self.tokenizer.decode(row[: int(n)].tolist()) for row, n in zip(t.responses.cpu(), t.seq_lens.cpu())]
        outputs = [fn(t.responses.cpu(), completions, t.answers) for fn in self.reward_functions]
        total = torch.stack([o.total_reward.float() for o in outputs]).sum(0).to(self.device)
        advantages = (total - total.mean()) / (total.std() + 1e-4) if total.numel() > 1 else total - total.mean()
        t.ref_logprobs, t.advantages, t.reward_outputs = ref_logprobs, advantages, outputs
        return t.to("cpu")

    def run(self, stop_event, max_groups: Optional[int] = None) -> None:
        while not stop_event.is_set() and (max_groups is None or self.groups_done < max_groups):
            try:
                traj = self.rollout_queue.get(timeout=0.2)
            except queue.Empty:
                continue
            done = self.process(traj)
            if not self.replay_buffer.extend(done, stop_event.is_set):
                return
            self.groups_done += 1
            if self.metric_logger is not None:
                payload: dict = {"postprocessing/groups": self.groups_done, "postprocessing/response_length": done.seq_lens.float().mean().item()}
                for o in done.reward_outputs:
                    payload.update(o.log(prefix="rewards"))
                self.metric_logger.log_dict(payload, step=self.groups_done)
