"""Proximal policy optimisation engine (single device, full fine-tune of policy and value model).

Reference behaviour: recipes/ppo_full_finetune_single_device.py:38-1240 — each step
(1) samples responses from the policy with a KV cache, (2) scores them with the frozen
reference policy, the value model and the frozen reward model, (3) forms KL-shaped rewards
and GAE advantages, (4) runs ``ppo_epochs`` passes of clipped-objective mini-batches over the
trajectory.  Config keys and logged metrics are the reference's.

Structure here: :class:`RolloutWorker` owns everything that runs without gradients (sampling
and scoring) and returns an :class:`~torchtune_b200.rlhf.Trajectory`; :class:`PPOTrainer` owns
optimisation and bookkeeping.
"""
from __future__ import annotations

import math
import time
from functools import partial
from typing import Any, Dict, List, Optional

import torch
from torch import nn
from tqdm import tqdm

from .. import config, generation, rlhf, training, utils
from ..config import DictConfig
from ..data import padded_collate
from ..rlhf import PPOStats, Trajectory
from .dataloading import StatefulDataLoader, StatefulDistributedSampler

log = utils.get_logger("DEBUG")


class RolloutWorker:
    """Sampling + scoring under ``torch.no_grad``."""

    def __init__(self, policy: nn.Module, ref_policy: nn.Module, value: nn.Module, reward: nn.Module, *, pad_id: int, stop_token_ids: torch.Tensor,
                 max_generated_tokens: int, temperature: float, top_k: Optional[int], enable_kv_cache: bool, penalise_no_eos: bool,
                 min_response_length: Optional[int], reward_penalty: float, rng: torch.Generator, dtype: torch.dtype):
        self.policy, self.ref_policy, self.value, self.reward = policy, ref_policy, value, reward
        self.pad_id, self.stop_token_ids = pad_id, stop_token_ids
        self.max_generated_tokens, self.temperature, self.top_k = max_generated_tokens, temperature, top_k
        self.enable_kv_cache = enable_kv_cache
        self.penalise_no_eos, self.min_response_length, self.reward_penalty = penalise_no_eos, min_response_length, reward_penalty
        self.rng, self.dtype = rng, dtype

    def _sample(self, input_ids: torch.Tensor):
        b, ctx = input_ids.shape
        if self.enable_kv_cache:
            self.policy.setup_caches(batch_size=b, dtype=self.dtype, decoder_max_seq_len=ctx + self.max_generated_tokens)
        try:
            return generation.generate(
                model=self.policy, prompt=input_ids, max_generated_tokens=self.max_generated_tokens, temperature=self.temperature,
                top_k=self.top_k, pad_id=self.pad_id, rng=self.rng,
            )
        finally:
            if self.enable_kv_cache:
                from ..modules.common_utils import delete_kv_caches

                delete_kv_caches(self.policy)

    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor) -> Trajectory:
        _, ctx = input_ids.shape
        query_responses, logits = self._sample(input_ids)
        responses = query_responses[:, ctx:].clone()
        not_pad = query_responses != self.pad_id
        masks = generation.get_causal_mask_from_padding_mask(not_pad)
        position_ids = generation.get_position_ids_from_padding_mask(not_pad)
        logprobs = rlhf.logits_to_logprobs(logits, responses, self.temperature)
        del logits
        ref_logits = rlhf.truncate_sequence_for_logprobs(self.ref_policy(query_responses, input_pos=position_ids, mask=masks), ctx)
        ref_logprobs = rlhf.logits_to_logprobs(ref_logits, responses, self.temperature)
        del ref_logits
        values = rlhf.truncate_sequence_for_logprobs(self.value(query_responses, input_pos=position_ids, mask=masks), ctx).squeeze(-1)
        response_padding_masks, responses = rlhf.truncate_sequence_at_first_stop_token(responses, self.stop_token_ids, self.pad_id)
        scores = self.reward(torch.cat([input_ids, responses], dim=1), input_pos=position_ids, mask=masks)
        seq_lens = training.get_unmasked_sequence_lengths(response_padding_masks)
        scores = scores.gather(1, (seq_lens + ctx)[:, None, None]).squeeze((-1, -2))
        if self.penalise_no_eos or self.min_response_length:
            penalty = rlhf.get_reward_penalty_mask(response_padding_masks, seq_lens, self.penalise_no_eos, self.min_response_length)
            scores[penalty] = self.reward_penalty
        logprobs[response_padding_masks] = 1.0
        ref_logprobs[response_padding_masks] = 1.0
        # the value of the token *after* the last response token is still meaningful
        value_seq_idxs = torch.where((seq_lens > 0) & (seq_lens < self.max_generated_tokens - 1), seq_lens + 1, seq_lens)
        value_padding_masks = response_padding_masks.clone().scatter_(1, value_seq_idxs.unsqueeze(-1), False)
        values[value_padding_masks] = 0.0
        return Trajectory(
            query_responses=query_responses, logprobs=logprobs, ref_logprobs=ref_logprobs, values=values, masks=masks, position_ids=position_ids,
            response_padding_masks=response_padding_masks, value_padding_masks=value_padding_masks, value_seq_idxs=value_seq_idxs, scores=scores, seq_lens=seq_lens,
        )

    def batched(self, input_ids: torch.Tensor, forward_batch_size: int) -> Trajectory:
        parts = [self(input_ids[i : i + forward_batch_size]) for i in range(0, input_ids.shape[0], forward_batch_size)]
        return Trajectory(*map(torch.cat, zip(*parts)))


class PPOTrainer:
    """Full fine-tuning of a policy and a value model against a frozen reward model."""

    def __init__(self, cfg: DictConfig) -> None:
        self.cfg = cfg
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(cfg.get("dtype"), device=self._device)
        if self._dtype == torch.float16:
            raise RuntimeError("full fp16 training is not supported with this recipe. Please use bf16 or fp32 instead.")
        self._output_dir = cfg.output_dir
        self._log_every_n_steps = cfg.get("log_every_n_steps", 1)
        self._log_peak_memory_stats = cfg.get("log_peak_memory_stats", False) and self._device.type == "cuda"
        self.seed = training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))
        self._rng = torch.Generator(self._device).manual_seed(self.seed)
        self._total_steps = 0
        self._steps_run = 0
        self._total_epochs = 0
        self._epochs_run = 0
        self.global_step = 0
        self._resume_from_checkpoint = cfg.get("resume_from_checkpoint", False)
        self._gradient_accumulation_steps = cfg.get("gradient_accumulation_steps", 1)
        self._optimizer_in_bwd = cfg.get("optimizer_in_bwd", False)
        if self._optimizer_in_bwd and self._gradient_accumulation_steps > 1:
            raise RuntimeError("Gradient accumulation is not supported with optimizer in bwd. Please set gradient_accumulation_steps=1, or optimizer_in_bwd=False.")

    # ------------------------------------------------------------------ setup
    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        self._metric_logger = config.instantiate(cfg.metric_logger)
        self._metric_logger.log_config(cfg)
        self._policy_checkpointer = config.instantiate(cfg.checkpointer, should_load_recipe_state=self._resume_from_checkpoint)
        ref_ckptr = config.instantiate(cfg.ref_policy_checkpointer, should_load_recipe_state=False)
        self._value_checkpointer = config.instantiate(cfg.value_checkpointer, should_load_recipe_state=False)
        reward_ckptr = config.instantiate(cfg.reward_checkpointer, should_load_recipe_state=False)
        policy_ckpt = self._policy_checkpointer.load_checkpoint()
        ref_sd = ref_ckptr.load_checkpoint()[training.MODEL_KEY]
        value_sd = self._value_checkpointer.load_checkpoint()[training.MODEL_KEY]
        reward_sd = reward_ckptr.load_checkpoint()[training.MODEL_KEY]
        self._setup_models(cfg, policy_ckpt[training.MODEL_KEY], ref_sd, value_sd, reward_sd)
        self._tokenizer = config.instantiate(cfg.tokenizer) if cfg.get("tokenizer") is not None else None
        self._pad_id = getattr(self._tokenizer, "pad_id", cfg.get("pad_id", 0)) if self._tokenizer is not None else cfg.get("pad_id", 0)
        self._optimizer = self._setup_optimizer(cfg.optimizer, policy_ckpt.get(training.OPT_KEY) if self._resume_from_checkpoint else None)
        self._loss_fn = config.instantiate(cfg.loss)
        self._dataloader = self._setup_data(cfg.dataset, cfg.shuffle, cfg.batch_size)
        self._setup_training_parameters(cfg)
        self._setup_training_hyperparameters(cfg)
        if self._resume_from_checkpoint:
            self._update_recipe_state(policy_ckpt)
        self._lr_scheduler = None
        if cfg.get("lr_scheduler") is not None and not self._optimizer_in_bwd:
            self._lr_scheduler = config.instantiate(cfg.lr_scheduler, self._optimizer, num_training_steps=self._total_steps * self._ppo_epochs * (self.batch_size // self._ppo_batch_size), last_epoch=self.global_step - 1)
        from ..training._profiler import DummyProfiler

        self._profiler = DummyProfiler()
        stop = cfg.get("stop_token_ids")
        if stop is None:
            stop = list(getattr(self._tokenizer, "stop_tokens", [])) if self._tokenizer is not None else []
        elif self._tokenizer is not None and hasattr(self._tokenizer, "stop_tokens") and not set(stop).issubset(set(self._tokenizer.stop_tokens)):
            import warnings

            warnings.warn(f"Stop tokens defined in `stop_token_ids` ({stop}) are not in the tokenizer's stop tokens ({self._tokenizer.stop_tokens}).")
        self._stop_token_ids = torch.tensor(list(stop), device=self._device, dtype=torch.long)
        self._rollout = RolloutWorker(
            self._policy_model, self._ref_policy_model, self._value_model, self._reward_model, pad_id=self._pad_id, stop_token_ids=self._stop_token_ids,
            max_generated_tokens=self._max_generated_tokens, temperature=self._temperature, top_k=self._top_k, enable_kv_cache=cfg.get("enable_kv_cache", True),
            penalise_no_eos=self._penalise_no_eos, min_response_length=self._min_response_length, reward_penalty=self._reward_penalty, rng=self._rng, dtype=self._dtype,
        )

    def _setup_models(self, cfg, policy_sd, ref_sd, value_sd, reward_sd) -> None:
        with training.set_default_dtype(self._dtype), self._device:
            self._policy_model = config.instantiate(cfg.policy_model)
            self._ref_policy_model = config.instantiate(cfg.policy_model)
            self._value_model = config.instantiate(cfg.reward_and_value_model)
            self._reward_model = config.instantiate(cfg.reward_and_value_model)
        if cfg.get("enable_activation_checkpointing", False):
            from .. import modules

            for m in (self._policy_model, self._value_model):
                training.set_activation_checkpointing(m, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
        self._policy_model.load_state_dict(policy_sd)
        self._ref_policy_model.load_state_dict(ref_sd)
        self._reward_model.load_state_dict(reward_sd)
        # a value model may start from a language-model or reward checkpoint: keep a fresh head
        # when the checkpoint's head has a different number of rows
        training.update_state_dict_for_classifier(value_sd, self._value_model.named_parameters())
        self._value_model.load_state_dict(value_sd)
        for m in (self._policy_model, self._value_model, self._ref_policy_model, self._reward_model):
            training.validate_expected_param_dtype(m.named_parameters(), dtype=self._dtype)
        for m in (self._ref_policy_model, self._reward_model):
            m.eval()
            for p in m.parameters():
                p.requires_grad_(False)
        training.disable_dropout(self._policy_model)
        training.disable_dropout(self._value_model)
        log.info(f"Models are initialized with precision {self._dtype}.")

    def _setup_optimizer(self, cfg_optimizer, opt_state):
        params = list(self._policy_model.parameters()) + list(self._value_model.parameters())
        if self._optimizer_in_bwd:
            optim_dict = {p: config.instantiate(cfg_optimizer, [p]) for p in params}
            training.register_optim_in_bwd_hooks(self._policy_model, optim_dict)
            training.register_optim_in_bwd_hooks(self._value_model, optim_dict)
            self._optim_ckpt_wrapper = _TwoModelOptimWrapper(self._policy_model, self._value_model, optim_dict)
            if opt_state is not None:
                self._optim_ckpt_wrapper.load_state_dict(opt_state)
            return None
        opt = config.instantiate(cfg_optimizer, params)
        if opt_state is not None:
            opt.load_state_dict(opt_state)
        log.info("Optimizer is initialized.")
        return opt

    def _setup_data(self, cfg_dataset, shuffle: bool, batch_size: int):
        ds = config.instantiate(cfg_dataset, self._tokenizer)
        sampler = StatefulDistributedSampler(ds, num_replicas=1, rank=0, shuffle=shuffle, seed=0)
        collate = partial(padded_collate, pad_direction="left", keys_to_pad=["tokens", "labels"], padding_idx=self._pad_id)
        return StatefulDataLoader(ds, batch_size=batch_size, sampler=sampler, collate_fn=collate, drop_last=True)

    def _setup_training_parameters(self, cfg) -> None:
        self.batch_size = cfg.batch_size
        self._forward_batch_size = cfg.forward_batch_size
        self._ppo_epochs = cfg.ppo_epochs
        self._ppo_batch_size = cfg.ppo_batch_size
        self._ppo_backward_batch_size = cfg.ppo_batch_size // self._gradient_accumulation_steps
        if self.batch_size % self._forward_batch_size != 0:
            raise ValueError(f"batch_size ({self.batch_size}) must be exactly divisible by forward_batch_size ({self._forward_batch_size}).")
        if self.batch_size % self._ppo_batch_size != 0:
            raise ValueError(f"batch_size ({self.batch_size}) must be exactly divisible by ppo_batch_size ({self._ppo_batch_size}).")
        if self._ppo_batch_size % self._gradient_accumulation_steps != 0:
            raise ValueError(f"ppo_batch_size ({self._ppo_batch_size}) must be exactly divisible by gradient_accumulation_steps ({self._gradient_accumulation_steps}).")
        self._total_steps = cfg.num_steps // self.batch_size
        batches_per_epoch = max(1, len(self._dataloader))
        self._total_epochs = math.ceil(self._total_steps / batches_per_epoch)
        if self._total_steps == 0:
            raise ValueError(f"num_steps {cfg.num_steps} must be greater than the batch size {self.batch_size}.")
        if self._total_steps < len(self._dataloader):
            import warnings

            warnings.warn(f"There are fewer total steps ({self._total_steps}, (num_steps//batch_size) than there are batches ({len(self._dataloader)}) in the dataset. Training will stop after ({self._total_steps}) steps without saving intermediate checkpoints")
        if self._total_steps > batches_per_epoch and self._total_steps % batches_per_epoch != 0:
            import warnings

            warnings.warn(f"num_steps ({cfg.num_steps}) is not exactly divisible by the number of batches in the dataset ({batches_per_epoch}). Intermediate checkpoints will only be saved every {batches_per_epoch} steps.")
        log.info(f"Total steps to run: {self._total_steps}, Total epochs to run: {self._total_epochs}")

    def _setup_training_hyperparameters(self, cfg) -> None:
        self._kl_coeff = cfg.kl_coeff
        self._gamma = cfg.gamma
        self._lmbda = cfg.lmbda
        self._whiten_rewards = cfg.get("whiten_rewards", False)
        self._temperature = cfg.temperature
        self._top_k = cfg.get("top_k")
        self._max_generated_tokens = cfg.max_generated_tokens
        self._min_response_length = cfg.get("min_response_length")
        self._penalise_no_eos = cfg.get("penalise_no_eos", False)
        self._reward_penalty = cfg.get("reward_penalty", -3)

    def _update_recipe_state(self, ckpt: Dict[str, Any]) -> None:
        try:
            if self.seed != ckpt[training.SEED_KEY] or self._total_steps != ckpt[training.MAX_STEPS_KEY] or self._total_epochs != ckpt[training.TOTAL_EPOCHS_KEY]:
                import warnings

                warnings.warn("Configured value for seed, total_steps, or total_epochs does not match the value stored in checkpoint.")
            self.seed = training.set_seed(seed=ckpt[training.SEED_KEY])
            self._rng.set_state(ckpt[training.RNG_KEY])
            self._steps_run = ckpt[training.STEPS_KEY]
            self._total_steps = ckpt[training.MAX_STEPS_KEY]
            self._total_epochs = ckpt[training.TOTAL_EPOCHS_KEY]
            self._epochs_run = ckpt[training.EPOCHS_KEY]
            self.global_step = ckpt.get("global_step", 0)
        except KeyError as exc:
            raise KeyError("Checkpoint does not contain the required keys needed for updating recipe state.Are you sure you passed in the right recipe checkpoint?") from exc

    # ------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, epoch: int, is_intermediate_checkpoint: bool = False) -> None:
        policy_ckpt: Dict[str, Any] = {training.MODEL_KEY: {k: v.detach().cpu() for k, v in self._policy_model.state_dict().items()}}
        value_ckpt: Dict[str, Any] = {training.MODEL_KEY: {k: v.detach().cpu() for k, v in self._value_model.state_dict().items()}}
        if is_intermediate_checkpoint:
            policy_ckpt.update(
                {
                    training.OPT_KEY: self._optim_ckpt_wrapper.state_dict() if self._optimizer_in_bwd else self._optimizer.state_dict(),
                    training.SEED_KEY: self.seed,
                    training.EPOCHS_KEY: self._epochs_run,
                    training.TOTAL_EPOCHS_KEY: self._total_epochs,
                    training.MAX_STEPS_KEY: self._total_steps,
                    training.STEPS_KEY: self._steps_run,
                    training.RNG_KEY: self._rng.get_state(),
                    "global_step": self.global_step,
                }
            )
        self._policy_checkpointer.save_checkpoint(policy_ckpt, epoch=epoch, intermediate_checkpoint=is_intermediate_checkpoint)
        self._value_checkpointer.save_checkpoint(value_ckpt, epoch=epoch, intermediate_checkpoint=False)

    # ------------------------------------------------------------------ train
    def train(self) -> None:
        if not self._optimizer_in_bwd:
            self._optimizer.zero_grad()
        done = False
        pbar = tqdm(total=self._total_steps, initial=self._steps_run)
        for curr_epoch in range(self._epochs_run, self._total_epochs):
            self._dataloader.sampler.set_epoch(curr_epoch)
            for batch in self._dataloader:
                tokens = batch["tokens"].to(self._device)
                ctx = tokens.shape[1]
                t0 = time.perf_counter()
                trajectory = self._rollout.batched(tokens, self._forward_batch_size)
                traj_time = time.perf_counter() - t0
                rewards, kl, kl_rewards = rlhf.get_rewards_ppo(trajectory.scores, trajectory.logprobs, trajectory.ref_logprobs, self._kl_coeff, trajectory.value_seq_idxs)
                if self._whiten_rewards:
                    rewards = rlhf.whiten(rewards, ~trajectory.response_padding_masks, shift_mean=True)  # unit variance, mean kept
                advantages, returns = rlhf.estimate_advantages(trajectory.values, rewards, self._gamma, self._lmbda, masks=~trajectory.response_padding_masks)
                t0 = time.perf_counter()
                stats: List[PPOStats] = []
                for _ in range(self._ppo_epochs):
                    order = torch.randperm(self.batch_size, device=self._device, generator=self._rng)
                    for i in range(0, self.batch_size, self._ppo_batch_size):
                        mini = order[i : i + self._ppo_batch_size]
                        micro_stats = []
                        for j in range(0, self._ppo_batch_size, self._ppo_backward_batch_size):
                            idxs = mini[j : j + self._ppo_backward_batch_size]
                            sub = Trajectory(*(t.index_select(0, idxs) for t in trajectory))
                            micro_stats.append(self.ppo_step(sub, advantages[idxs], returns[idxs], ctx))
                        stats.append(PPOStats(*map(sum, zip(*micro_stats))))
                        if not self._optimizer_in_bwd:
                            self._optimizer.step()
                            self._optimizer.zero_grad(set_to_none=True)
                        if self._lr_scheduler is not None:
                            self._lr_scheduler.step()
                        self.global_step += 1
                ppo_time = time.perf_counter() - t0
                self._steps_run += 1
                if self._steps_run % self._log_every_n_steps == 0:
                    lr = training.get_lr(self._optimizer if not self._optimizer_in_bwd else self._optim_ckpt_wrapper)
                    self.log_metrics(trajectory, PPOStats(*map(torch.stack, zip(*stats))), kl, kl_rewards, tokens.numel() / traj_time, tokens.numel() / ppo_time, lr)
                del trajectory, stats, advantages, returns, kl, kl_rewards
                pbar.update(1)
                if self._steps_run == self._total_steps:
                    done = True
                    break
            self._epochs_run += 1
            self.save_checkpoint(curr_epoch, is_intermediate_checkpoint=not done)
            if done:
                return

    def ppo_step(self, trajectory: Trajectory, advantages: torch.Tensor, returns: torch.Tensor, context_length: int) -> PPOStats:
        pi_logits = self._policy_model(trajectory.query_responses, input_pos=trajectory.position_ids, mask=trajectory.masks)
        pi_logits = rlhf.truncate_sequence_for_logprobs(pi_logits, context_length)
        pi_logprobs = rlhf.logits_to_logprobs(pi_logits, trajectory.query_responses[:, context_length:], self._temperature)
        pi_logprobs = pi_logprobs.masked_fill(trajectory.response_padding_masks, 1.0)
        del pi_logits
        phi_values = self._value_model(trajectory.query_responses, input_pos=trajectory.position_ids, mask=trajectory.masks)
        phi_values = rlhf.truncate_sequence_for_logprobs(phi_values, context_length).squeeze(-1)
        phi_values = phi_values.masked_fill(trajectory.value_padding_masks, 0.0)
        loss, policy_loss, value_loss, ratios, clipfrac = self._loss_fn(
            trajectory.logprobs, pi_logprobs, advantages, trajectory.values, phi_values, returns,
            padding_masks=~trajectory.response_padding_masks, value_padding_masks=~trajectory.value_padding_masks,
        )
        ga = self._gradient_accumulation_steps
        loss = loss / ga
        loss.backward()
        with torch.no_grad():
            approx_kl = (0.5 * (pi_logprobs - trajectory.logprobs).pow(2)).mean()
        return PPOStats(loss.detach(), policy_loss / ga, value_loss / ga, ratios / ga, clipfrac / ga, approx_kl / ga)

    def log_metrics(self, trajectory: Trajectory, ppo_stats: PPOStats, kl, kl_rewards, tps_traj: float, tps_ppo: float, lr: float) -> None:
        log_dict = {
            "scores": trajectory.scores.mean(),
            "num_stop_tokens": trajectory.response_padding_masks.any(-1).sum(),
            "rlhf_reward": trajectory.scores.mean() + kl_rewards.sum(1).mean(),
            "kl": kl.sum(1).mean(),
            "kl_reward": kl_rewards.sum(1).mean(),
            "lr": lr,
            "loss": ppo_stats.loss.mean(),
            "policy_loss": ppo_stats.policy_loss.mean(),
            "value_loss": ppo_stats.value_loss.mean(),
            "clipfrac": ppo_stats.clipfrac.mean(),
            "ratios": ppo_stats.ratios.mean(),
            "approx_policy_kl": ppo_stats.approx_policy_kls.mean(),
            "response_lengths": trajectory.seq_lens.float().mean(),
            "tokens_per_second_per_gpu_trajectory": tps_traj,
            "tokens_per_second_per_gpu_ppo": tps_ppo,
        }
        log_dict = {k: (v.item() if isinstance(v, torch.Tensor) else v) for k, v in log_dict.items()}
        if self._log_peak_memory_stats:
            log_dict.update(training.get_memory_stats(device=self._device))
        self._metric_logger.log_dict(log_dict, step=self.global_step)

    def cleanup(self) -> None:
        self._metric_logger.close()


class _TwoModelOptimWrapper:
    """Checkpoint view over per-parameter optimizers that span the policy and the value model."""

    def __init__(self, policy: nn.Module, value: nn.Module, optim_dict: Dict[nn.Parameter, torch.optim.Optimizer]):
        self.optim_map = {}
        for prefix, model in (("policy", policy), ("value", value)):
            for name, p in model.named_parameters():
                if p in optim_dict:
                    self.optim_map[f"{prefix}.{name}"] = optim_dict[p]

    def state_dict(self) -> Dict[str, Any]:
        return {k: o.state_dict() for k, o in self.optim_map.items()}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        missing = set(self.optim_map) ^ set(sd)
        if missing:
            raise RuntimeError(f"optimizer checkpoint keys do not match the models: {sorted(missing)[:5]}")
        for k, o in self.optim_map.items():
            o.load_state_dict(sd[k])

    def get_optim_key(self, key: str) -> Any:
        return next(iter(self.optim_map.values())).param_groups[0][key]
