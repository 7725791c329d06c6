"""Training role (parity: torchtune/dev/rl/workers/trainers/training.py:35-925): optimise the policy on groups from the replay
buffer and publish the weights every ``steps_before_weight_sync`` steps."""
from __future__ import annotations

import time
from typing import Any, Dict, Optional

import torch
from torch import nn

from .... import generation
from ..datatypes import Trajectory
from ..types import GRPOStats
from .parameter_servers import ParameterServer
from .replay import ReplayBuffer


class TrainingWorker:
    def __init__(self, *, model: nn.Module, optimizer, loss_fn, replay_buffer: ReplayBuffer, param_server: Optional[ParameterServer], device: torch.device, batch_groups: int,
                 num_steps: int, ppo_epochs: int = 1, clip_grad_norm: Optional[float] = None, steps_before_weight_sync: int = 1, metric_logger=None, pad_id: int = 0, parallel=None,
                 save_fn=None, save_every_n_steps: Optional[int] = None, activations_ctx=None):
        self.model, self.optimizer, self.loss_fn, self.replay_buffer, self.param_server = model, optimizer, loss_fn, replay_buffer, param_server
        self.device, self.batch_groups, self.num_steps, self.ppo_epochs = device, batch_groups, num_steps, ppo_epochs
        self.clip_grad_norm, self.steps_before_weight_sync = clip_grad_norm, max(1, steps_before_weight_sync)
        self.metric_logger, self.pad_id, self.parallel, self.save_fn, self.save_every_n_steps, self.activations_ctx = metric_logger, pad_id, parallel, save_fn, save_every_n_steps, activations_ctx
        self.loss_fn.set_model_output(model)
        self.step = 0
        self.policy_version = 0
        self.history: list = []

    def _state_dict(self) -> Dict[str, torch.Tensor]:
        if self.parallel is not None:
            return self.parallel.gather_full_state_dict(self.model)
        return {k: v.detach() for k, v in self.model.state_dict().items()}

    def grpo_step(self, traj: Trajectory) -> GRPOStats:
        t = traj.to(self.device)
        ctx = t.query_responses.shape[1] - t.responses.shape[1]
        masks = generation.get_causal_mask_from_padding_mask(t.query_response_padding_masks)
        position_ids = generation.get_position_ids_from_padding_mask(t.query_response_padding_masks)
        keep = t.query_response_padding_masks[:, ctx:]
        if self.activations_ctx is not None:
            with self.activations_ctx:
                hidden = self.model(t.query_responses, input_pos=position_ids, mask=masks)
        else:
            hidden = self.model(t.query_responses, input_pos=position_ids, mask=masks)
        hidden = hidden[:, ctx - 1 : -1]  # the state at position i predicts token i + 1
        loss, policy_loss, kl_loss, ratios, clipfrac, pi_logprobs = self.loss_fn(hidden, t.responses, t.ref_logprobs, t.advantages, padding_masks=keep)
        loss.backward()
        grad_norm = None
        if self.parallel is not None:
            grad_norm = self.parallel.optimizer_step(self.model, self.optimizer, 1.0 / self.parallel.dp_size, self.clip_grad_norm)
        else:
            if self.clip_grad_norm is not None:
                grad_norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), max_norm=float(self.clip_grad_norm))
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
        with torch.no_grad():
            m = keep.float()
            approx_kl = (0.5 * (pi_logprobs - t.logprobs).pow(2) * m).sum() / m.sum().clamp(min=1)
        return GRPOStats(loss.detach(), policy_loss, kl_loss, ratios, clipfrac, approx_kl, metadata={"grad_norm": grad_norm})

    def publish(self) -> None:
        if self.param_server is None:
            return
        sd = self._state_dict()  # collective under data parallelism: every trainer rank takes part, rank 0 publishes
        if self.parallel is None or self.parallel.rank == 0:
            self.policy_version = self.param_server.publish(sd)

    def run(self, stop_event) -> None:
        """``num_steps`` optimisation steps, then raise the stop flag for every other role."""
        try:
            while self.step < self.num_steps and not stop_event.is_set():
                t0 = time.perf_counter()
                traj = self.replay_buffer.sample(self.batch_groups, stop_event.is_set, pad_id=self.pad_id)
                if traj is None:
                    break
                waited = time.perf_counter() - t0
                t0 = time.perf_counter()
                stats = [self.grpo_step(traj) for _ in range(self.ppo_epochs)]
                self.step += 1
                if self.step % self.steps_before_weight_sync == 0:
                    self.publish()
                if self.save_fn is not None and self.save_every_n_steps and self.step % self.save_every_n_steps == 0:
                    self.save_fn(self, self.step)
                mean = lambda name: torch.stack([getattr(s, name).float().cpu() for s in stats]).mean().item()  # noqa: E731
                payload: Dict[str, Any] = {
                    "train/loss": mean("loss"), "train/policy_loss": mean("policy_loss"), "train/kl_loss": mean("kl_loss"), "train/approx_policy_kl": mean("approx_policy_kls"),
                    "train/policy_staleness": self.policy_version - traj.policy_version, "train/time_waiting_for_data_s": waited, "train/time_step_s": time.perf_counter() - t0,
                    "train/tokens_per_second": traj.query_responses.numel() * self.ppo_epochs / max(time.perf_counter() - t0, 1e-9),
                }
                gn = stats[-1].metadata.get("grad_norm") if stats[-1].metadata else None
                if gn is not None:
                    payload["train/grad_norm"] = float(gn)
                self.history.append(payload)
                if self.metric_logger is not None:
                    self.metric_logger.log_dict(payload, step=self.step)
        finally:
            stop_event.set()
