"""Group-relative policy optimisation engine (synchronous; one device or data parallel).

Reference behaviour: recipes/dev/grpo_full_finetune_distributed.py:60-1100 — every step draws ``batch_size`` prompts, samples
``grpo_samples`` completions per prompt from the current policy, scores them with a rule-based reward, normalises the rewards inside
each prompt's group into advantages, and runs ``ppo_epochs`` optimisation passes of a GRPO loss with a KL term against a frozen
reference policy.  Logged: ``loss, policy_loss, kl_loss, ratios, clipfrac, approx_policy_kl, rewards, successes, response_lengths``.

Under ``tune run --nproc_per_node N`` each rank works on its own prompts and gradients go through the resident data-parallel
engine (fused reduce → AdamW → broadcast); generation needs no weight synchronisation because parameters are resident on every rank.
"""
from __future__ import annotations

import time
from functools import partial
from typing import Any, Dict, List, Optional

import torch
from torch import nn
from tqdm import tqdm

from .. import config, generation, rlhf, training, utils
from ..config import DictConfig
from ..config._resolve import get_component_from_path
from ..dev.grpo import GRPOStats, GRPOTrajectory, batch_shaped_correctness_reward, padded_collate_rl
from ..modules.common_utils import delete_kv_caches
from .dataloading import StatefulDataLoader, StatefulDistributedSampler

log = utils.get_logger("DEBUG")


def _left_pad(tokens: torch.Tensor, pad_id: int) -> torch.Tensor:
    """Right-padded ``[b, s]`` → left-padded (generation appends at the right end of every row)."""
    out = torch.full_like(tokens, pad_id)
    lens = (tokens != pad_id).sum(1)
    for i, n in enumerate(lens.tolist()):
        if n:
            out[i, tokens.shape[1] - n :] = tokens[i, :n]
    return out


class GRPOTrainer:
    def __init__(self, cfg: DictConfig, *, distributed: bool = False) -> None:
        self.cfg = cfg
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(cfg.get("dtype"), device=self._device)
        self.parallel = None
        if distributed:
            from .. import parallel

            self.parallel = parallel.init_from_config(cfg, self._device)
        self.world_size, self.rank = utils.get_world_size_and_rank()
        self._is_rank_zero = self.rank == 0
        self._output_dir = cfg.output_dir
        self._log_every_n_steps = cfg.get("log_every_n_steps", 1)
        self._log_peak_memory_stats = cfg.get("log_peak_memory_stats", False) and self._device.type == "cuda"
        self.seed = training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))
        self._rng = torch.Generator(self._device).manual_seed(self.seed)
        self._resume_from_checkpoint = cfg.get("resume_from_checkpoint", False)
        self._clip_grad_norm = cfg.get("clip_grad_norm")
        self._steps_run = 0
        self._epochs_run = 0
        self.global_step = 0

    # ------------------------------------------------------------------ setup
    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        if self._is_rank_zero:
            self._metric_logger = config.instantiate(cfg.metric_logger)
            self._metric_logger.log_config(cfg)
        self._checkpointer = config.instantiate(cfg.checkpointer, should_load_recipe_state=self._resume_from_checkpoint)
        ckpt = self._checkpointer.load_checkpoint()
        ref_sd = config.instantiate(cfg.ref_checkpointer, should_load_recipe_state=False).load_checkpoint()[training.MODEL_KEY]
        with training.set_default_dtype(self._dtype), self._device:
            self._model = config.instantiate(cfg.model)
            self._ref_model = config.instantiate(cfg.model)
        if cfg.get("enable_activation_checkpointing", False):
            from .. import modules

            training.set_activation_checkpointing(self._model, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
        self._ref_model.load_state_dict(ref_sd)
        self._ref_model.eval()
        for p in self._ref_model.parameters():
            p.requires_grad_(False)
        if self.parallel is not None:
            self._model = self.parallel.shard_model(self._model, cfg, ckpt[training.MODEL_KEY], None, dtype=self._dtype, strict=True)
        else:
            self._model.load_state_dict(ckpt[training.MODEL_KEY])
        training.disable_dropout(self._model)
        self._tokenizer = config.instantiate(cfg.tokenizer)
        self._pad_id = getattr(self._tokenizer, "pad_id", 0)
        opt_state = ckpt.get(training.OPT_KEY) if self._resume_from_checkpoint else None
        if self.parallel is not None:
            self._optimizer = self.parallel.build_optimizer(self._model, cfg.optimizer, opt_state)
        else:
            self._optimizer = config.instantiate(cfg.optimizer, list(self._model.parameters()))
            if opt_state is not None:
                self._optimizer.load_state_dict(opt_state)
        self._loss_fn = config.instantiate(cfg.loss)
        reward_fn = cfg.get("reward_fn")
        self._reward_fn = get_component_from_path(reward_fn) if reward_fn else batch_shaped_correctness_reward

        ds = config.instantiate(cfg.dataset, self._tokenizer)
        dp_size = self.parallel.dp_size if self.parallel is not None else 1
        dp_rank = self.parallel.dp_rank if self.parallel is not None else 0
        sampler = StatefulDistributedSampler(ds, num_replicas=dp_size, rank=dp_rank, shuffle=cfg.get("shuffle", True), seed=self.seed)
        self._dataloader = StatefulDataLoader(ds, batch_size=cfg.batch_size, sampler=sampler, collate_fn=partial(padded_collate_rl, padding_idx=self._pad_id), drop_last=True)

        self.batch_size = cfg.batch_size
        self.grpo_samples = cfg.grpo_samples
        self._forward_batch_size = cfg.get("forward_batch_size", cfg.batch_size * cfg.grpo_samples)
        self._ppo_epochs = cfg.get("ppo_epochs", 1)
        self._max_generated_tokens = cfg.max_generated_tokens
        self._temperature = cfg.get("temperature", 1.0)
        self._top_k = cfg.get("top_k")
        self._total_steps = cfg.num_steps
        self._total_epochs = cfg.get("epochs", 1)
        self._save_every_n_epochs = cfg.get("save_every_n_epochs", 1)
        stop = cfg.get("stop_token_ids") or list(getattr(self._tokenizer, "stop_tokens", []))
        self._stop_token_ids = torch.tensor(list(stop), device=self._device, dtype=torch.long)
        if self._resume_from_checkpoint:
            self._steps_run = ckpt.get(training.STEPS_KEY, 0)
            self._epochs_run = ckpt.get(training.EPOCHS_KEY, 0)
            if training.RNG_KEY in ckpt:
                self._rng.set_state(ckpt[training.RNG_KEY])
        self._lr_scheduler = None
        if cfg.get("lr_scheduler") is not None:
            target = getattr(self._optimizer, "torch_optimizer", self._optimizer)
            self._lr_scheduler = config.instantiate(cfg.lr_scheduler, target, num_training_steps=self._total_steps * self._ppo_epochs, last_epoch=self.global_step - 1)

    # ------------------------------------------------------------------ rollout
    def _response_logprobs(self, model: nn.Module, query_responses, masks, position_ids, ctx: int) -> torch.Tensor:
        logits = model(query_responses, input_pos=position_ids, mask=masks)
        logits = rlhf.truncate_sequence_for_logprobs(logits, ctx)
        return rlhf.logits_to_logprobs(logits, query_responses[:, ctx:], self._temperature)

    @torch.no_grad()
    def generate_trajectory(self, prompts: torch.Tensor, answers: List[str]) -> GRPOTrajectory:
        b, ctx = prompts.shape
        g = self.grpo_samples
        batch = _left_pad(prompts, self._pad_id)[:, None, :].expand(b, g, ctx).reshape(b * g, ctx)
        self._model.setup_caches(batch_size=b * g, dtype=self._dtype, decoder_max_seq_len=ctx + self._max_generated_tokens)
        try:
            query_responses, _ = generation.generate(model=self._model, prompt=batch, max_generated_tokens=self._max_generated_tokens, temperature=self._temperature, top_k=self._top_k,
                                                     pad_id=self._pad_id, rng=self._rng, stop_tokens=self._stop_token_ids.tolist() or None,
                                                     return_logits=False)  # log-probabilities are recomputed below; no [b, n, vocab] tensor is kept
        finally:
            delete_kv_caches(self._model)
        not_pad = query_responses != self._pad_id
        masks = generation.get_causal_mask_from_padding_mask(not_pad)
        position_ids = generation.get_position_ids_from_padding_mask(not_pad)
        responses = query_responses[:, ctx:].clone()
        logprobs = self._response_logprobs(self._model, query_responses, masks, position_ids, ctx)
        ref_logprobs = self._response_logprobs(self._ref_model, query_responses, masks, position_ids, ctx)
        response_padding_masks, responses = rlhf.truncate_sequence_at_first_stop_token(responses, self._stop_token_ids, self._pad_id)
        seq_lens = training.get_unmasked_sequence_lengths(response_padding_masks)
        rewards, successes = self._reward_fn(self._tokenizer, responses.reshape(b, g, -1).cpu(), answers)
        rewards, successes = rewards.to(self._device), successes.to(self._device)
        advantages = (rewards - rewards.mean(1, keepdim=True)) / (rewards.std(1, keepdim=True) + 1e-4) if g > 1 else rewards - rewards.mean()
        logprobs[response_padding_masks] = 1.0
        ref_logprobs[response_padding_masks] = 1.0
        self._last_rewards, self._last_successes = rewards, successes
        return GRPOTrajectory(query_responses=query_responses, logprobs=logprobs, ref_logprobs=ref_logprobs, advantages=advantages.reshape(b * g), masks=masks, position_ids=position_ids,
                              response_padding_masks=response_padding_masks, seq_lens=seq_lens, answers=answers)

    # ------------------------------------------------------------------ optimisation
    def grpo_step(self, traj: GRPOTrajectory, ctx: int) -> GRPOStats:
        n = traj.query_responses.shape[0]
        chunks = max(1, -(-n // self._forward_batch_size))
        totals = None
        for idx in torch.arange(n, device=self._device).tensor_split(chunks):
            pi = self._response_logprobs(self._model, traj.query_responses[idx], traj.masks[idx], traj.position_ids[idx], ctx)
            pad = traj.response_padding_masks[idx]
            pi = pi.masked_fill(pad, 1.0)
            loss, policy_loss, kl_loss, ratios, clipfrac = self._loss_fn(traj.logprobs[idx], pi, traj.ref_logprobs[idx], traj.advantages[idx], padding_masks=~pad)
            (loss * (idx.numel() / n)).backward()
            with torch.no_grad():
                approx_kl = (0.5 * (pi - traj.logprobs[idx]).pow(2)).mean()
            part = [t.detach().float().to(self._device) * (idx.numel() / n) for t in (loss, policy_loss, kl_loss, ratios, clipfrac, approx_kl)]
            totals = part if totals is None else [a + b for a, b in zip(totals, part)]
        grad_norm = None
        if self.parallel is not None:
            grad_norm = self.parallel.optimizer_step(self._model, self._optimizer, 1.0 / self.parallel.dp_size, self._clip_grad_norm)
        else:
            if self._clip_grad_norm is not None:
                grad_norm = torch.nn.utils.clip_grad_norm_(self._model.parameters(), max_norm=float(self._clip_grad_norm))
            self._optimizer.step()
            self._optimizer.zero_grad(set_to_none=True)
        if self._lr_scheduler is not None:
            self._lr_scheduler.step()
        self.global_step += 1
        return GRPOStats(*totals, metadata={"grad_norm": grad_norm})

    def train(self) -> None:
        if hasattr(self._optimizer, "zero_grad"):
            self._optimizer.zero_grad()
        pbar = tqdm(total=self._total_steps, initial=self._steps_run, disable=not self._is_rank_zero)
        done = False
        for epoch in range(self._epochs_run, self._total_epochs):
            self._dataloader.sampler.set_epoch(epoch)
            for batch in self._dataloader:
                tokens = batch["tokens"].to(self._device)
                ctx = tokens.shape[1]
                t0 = time.perf_counter()
                traj = self.generate_trajectory(tokens, batch["answers"])
                t_traj = time.perf_counter() - t0
                t0 = time.perf_counter()
                stats = [self.grpo_step(traj, ctx) for _ in range(self._ppo_epochs)]
                t_opt = time.perf_counter() - t0
                self._steps_run += 1
                if self._steps_run % self._log_every_n_steps == 0:
                    self.log_metrics(traj, stats, t_traj, t_opt)
                pbar.update(1)
                if self._steps_run >= self._total_steps:
                    done = True
                    break
            self._epochs_run += 1
            if done or self._epochs_run % self._save_every_n_epochs == 0:
                self.save_checkpoint(epoch, intermediate=not done)
            if done:
                break

    def log_metrics(self, traj: GRPOTrajectory, stats: List[GRPOStats], t_traj: float, t_opt: float) -> None:
        mean = lambda name: torch.stack([getattr(s, name) for s in stats]).mean()  # noqa: E731
        vals = {
            "loss": mean("loss"), "policy_loss": mean("policy_loss"), "kl_loss": mean("kl_loss"), "ratios": mean("ratios"), "clipfrac": mean("clipfrac"), "approx_policy_kl": mean("approx_policy_kls"),
            "rewards": self._last_rewards.mean(), "successes": self._last_successes.mean(), "response_lengths": traj.seq_lens.float().mean(),
        }
        keys = sorted(vals)
        packed = torch.stack([vals[k].float().to(self._device) for k in keys])
        if self.parallel is not None:
            self.parallel.all_reduce_sum_(packed)
            packed = packed / self.world_size
        if not self._is_rank_zero:
            return
        out = {k: v.item() for k, v in zip(keys, packed)}
        n_tokens = traj.query_responses.numel()
        out.update({"lr": training.get_lr(self._optimizer), "tokens_per_second_per_gpu_trajectory": n_tokens / t_traj, "tokens_per_second_per_gpu_grpo": n_tokens * self._ppo_epochs / t_opt})
        gn = stats[-1].metadata.get("grad_norm") if stats[-1].metadata else None
        if gn is not None:
            out["grad_norm"] = float(gn)
        if self._log_peak_memory_stats:
            out.update(training.get_memory_stats(device=self._device))
        self._metric_logger.log_dict(out, step=self.global_step)

    def save_checkpoint(self, epoch: int, intermediate: bool) -> None:
        if self.parallel is not None:
            model_sd = self.parallel.gather_full_state_dict(self._model)
            opt_sd = self.parallel.gather_optimizer_state_dict(self._model, self._optimizer) if intermediate else None
        else:
            model_sd = {k: v.detach().cpu() for k, v in self._model.state_dict().items()}
            opt_sd = self._optimizer.state_dict() if intermediate else None
        if self._is_rank_zero:
            ckpt: Dict[str, Any] = {training.MODEL_KEY: model_sd}
            if intermediate:
                ckpt.update({training.OPT_KEY: opt_sd, training.SEED_KEY: self.seed, training.EPOCHS_KEY: self._epochs_run, training.TOTAL_EPOCHS_KEY: self._total_epochs,
                             training.MAX_STEPS_KEY: self._total_steps, training.STEPS_KEY: self._steps_run, training.RNG_KEY: self._rng.get_state()})
            self._checkpointer.save_checkpoint(ckpt, epoch=epoch, intermediate_checkpoint=intermediate)
        if self.parallel is not None:
            self.parallel.barrier()

    def cleanup(self) -> None:
        if self._is_rank_zero:
            self._metric_logger.close()
        if self.parallel is not None:
            self.parallel.shutdown()
