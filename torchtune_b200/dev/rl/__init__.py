"""Asynchronous reinforcement learning from rule-based rewards: the roles of the reference's Ray + vLLM prototype
(torchtune/dev/rl, recipes/dev/async_grpo_full_finetune_distributed.py:118-315) rebuilt on this framework's own generator and
plain Python queues, so the topology runs (and is tested) without either package.

Roles, each a worker object driven by its own thread or process:

* :class:`workers.SyncLLMCollector` — holds a copy of the policy, samples ``group_size`` completions per prompt and puts
  :class:`datatypes.Trajectory` objects on the rollout queue; picks up newer weights from the parameter server between batches;
* :class:`workers.PostProcessingWorker` — reference-policy log-probabilities, rewards and group-relative advantages; fills the
  replay buffer;
* :class:`workers.TrainingWorker` — samples the replay buffer, optimises :class:`linear_grpo_loss.LinearGRPOLoss` and publishes
  its weights every ``steps_before_weight_sync`` steps;
* :class:`workers.ParameterServer` — the latest published weights and their version;
* :class:`workers.MetricLoggerWorker` — one logger behind a queue for all roles.
"""
from .linear_grpo_loss import LinearGRPOLoss
from .types import GRPOStats, GRPOTrajectory

__all__ = ["GRPOStats", "GRPOTrajectory", "LinearGRPOLoss"]
