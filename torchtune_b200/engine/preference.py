"""Direct preference optimisation engine (LoRA and full, single device and distributed).

Reference behaviour: recipes/lora_dpo_single_device.py:38-640,
recipes/lora_dpo_distributed.py:47-800, recipes/full_dpo_distributed.py:53-1100 — a batch is
``2B`` sequences (chosen then rejected); policy and reference sequence log-probabilities go
through a preference loss; rewards, accuracies, margins and mean log-probs / logits are logged.

Differences by design: the sequence log-probabilities are computed by the fused
``hidden → logits → log-softmax → gather`` operator (:func:`torchtune_b200.ops.token_logprobs`),
so the ``[2B, L, vocab]`` logits are never materialised — not for the policy, and not for the
reference pass either; the logged mean logit is obtained exactly from
``mean_t(h_t) · mean_v(W_v)``.  For LoRA runs the reference model is the policy with adapters
switched off; full DPO loads a frozen copy from ``ref_checkpointer``.
"""
from __future__ import annotations

import time
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn
from tqdm import tqdm

from .. import config, ops, rlhf, training, utils
from ..config import DictConfig
from ..data import CROSS_ENTROPY_IGNORE_IDX, padded_collate_dpo
from ..modules.peft import disable_adapter
from ..rlhf import ChosenRejectedOutputs
from .sft import SFTTrainer
from .timing import StepTimer

log = utils.get_logger("DEBUG")


def _plain_projection(proj: nn.Module) -> Optional[torch.Tensor]:
    """Weight of an output projection the fused log-prob operator can consume directly."""
    if hasattr(proj, "adapter_params") or getattr(proj, "bias", None) is not None:
        return None
    w = getattr(proj, "weight", None)
    if w is None and hasattr(proj, "tied_module"):
        w = proj.tied_module.weight
    return w if isinstance(w, torch.Tensor) and w.dim() == 2 else None


def sequence_logprobs(model: nn.Module, tokens: torch.Tensor, labels: torch.Tensor, ignore_index: int = CROSS_ENTROPY_IGNORE_IDX, **fwd) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(sum_t log p(label_t), mean logit)`` per sequence; labels are shifted left by one as in
    torchtune/rlhf/sequence_processing.py:138-178."""
    core = getattr(model, "decoder", model)
    weight = _plain_projection(core.output) if hasattr(core, "output") else None
    if weight is None:
        prev = getattr(core, "skip_output_layer", False)
        core.skip_output_layer = False
        try:
            logits = model(tokens, **fwd)
        finally:
            core.skip_output_layer = prev
        return rlhf.get_batch_log_probs(logits, labels, label_pad_token_id=ignore_index), logits.detach().float().mean(dim=(1, 2))
    prev = getattr(core, "skip_output_layer", False)
    core.skip_output_layer = True
    try:
        hidden = model(tokens, **fwd)
    finally:
        core.skip_output_layer = prev
    per_token = ops.token_logprobs(hidden[:, :-1].contiguous(), weight, labels[:, 1:].contiguous(), ignore_index, softcap=ops.logit_softcap_of(core))
    with torch.no_grad():
        mean_logit = hidden.detach().float().mean(dim=1) @ weight.detach().float().mean(dim=0)
    return per_token.sum(-1), mean_logit


class PreferenceStep:
    """One preference-optimisation step on a batch that already lives on the device: concatenated policy forward, reference
    forward (a frozen ``ref_model``, or the policy itself with its adapters switched off), preference loss, backward, update.

    ``tokens`` / ``labels`` are ``[2B, L]`` with the chosen sequences first (recipes/lora_dpo_distributed.py:592-640).  The
    returned loss is the mean over this rank's pairs (a device scalar; nothing is read back here).  With a ``parallel`` engine
    the gradients are averaged over its data-parallel ranks by the engine's fused update.
    """

    def __init__(self, model: nn.Module, loss_fn, optimizer, device: torch.device, parallel=None, ref_model: Optional[nn.Module] = None,
                 clip_grad_norm: Optional[float] = None, activations_ctx=None):
        self.model, self.loss_fn, self.optimizer, self.device = model, loss_fn, optimizer, device
        self.parallel, self.ref_model, self.clip_grad_norm = parallel, ref_model, clip_grad_norm
        self.activations_ctx = activations_ctx
        self._params = [p for p in model.parameters() if p.requires_grad]
        self.last_stats: Dict[str, torch.Tensor] = {}

    def upload(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def _logps(self, model: nn.Module, tokens: torch.Tensor, labels: torch.Tensor) -> ChosenRejectedOutputs:
        n = tokens.shape[0] // 2
        if self.activations_ctx is not None:
            with self.activations_ctx:
                logps, _ = sequence_logprobs(model, tokens, labels)
        else:
            logps, _ = sequence_logprobs(model, tokens, labels)
        return ChosenRejectedOutputs(chosen_logps=logps[:n], rejected_logps=logps[n:])

    def reference(self, tokens: torch.Tensor, labels: torch.Tensor) -> ChosenRejectedOutputs:
        if getattr(self.loss_fn, "is_reference_free", lambda: False)() is True:
            return ChosenRejectedOutputs(None, None)
        with torch.no_grad():
            if self.ref_model is not None:
                return self._logps(self.ref_model, tokens, labels)
            with disable_adapter(self.model):
                return self._logps(self.model, tokens, labels)

    def compute(self, batch: Dict[str, Any]) -> torch.Tensor:
        tokens, labels = batch["tokens"], batch["labels"]
        policy = self._logps(self.model, tokens, labels)
        reference = self.reference(tokens, labels)
        losses, chosen_rewards, rejected_rewards = self.loss_fn(policy, reference)
        loss = losses.mean()
        loss.backward()
        self.last_stats = {"rewards/chosen": chosen_rewards.mean(), "rewards/rejected": rejected_rewards.mean(),
                           "rewards/accuracies": (chosen_rewards > rejected_rewards).float().mean()}
        if self.parallel is not None:
            self.parallel.optimizer_step(self.model, self.optimizer, 1.0 / self.parallel.dp_size, self.clip_grad_norm)
        else:
            if self.clip_grad_norm is not None:
                torch.nn.utils.clip_grad_norm_(self._params, max_norm=float(self.clip_grad_norm))
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
        return loss.detach()

    def __call__(self, host_batch: Dict[str, Any]) -> torch.Tensor:
        return self.compute(self.upload(host_batch))


class DPOTrainer(SFTTrainer):
    def __init__(self, cfg: DictConfig, *, distributed: bool = False, lora: bool = True) -> None:
        super().__init__(cfg, distributed=distributed, lora=lora)
        self._ref_model: Optional[nn.Module] = None
        if self._optimizer_in_bwd:
            raise RuntimeError("optimizer_in_bwd is not supported by the preference-optimisation recipes")

    # ------------------------------------------------------------------ setup
    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        if self._is_rank_zero:
            self._metric_logger = config.instantiate(cfg.metric_logger)
            self._metric_logger.log_config(cfg)
        ckpt = self.load_checkpoint(cfg.checkpointer)
        self._loss_fn = config.instantiate(cfg.loss)
        self._model = self._setup_model(cfg, ckpt)
        if not self.is_lora:
            self._ref_model = self._setup_reference_model(cfg)
        self._tokenizer = config.instantiate(cfg.tokenizer) if cfg.get("tokenizer") is not None else None
        self._optimizer = self._setup_optimizer(cfg.optimizer, ckpt.get(training.OPT_KEY) if self._resume_from_checkpoint else None)
        utils.log_rank_zero(log, "Loss is initialized.")
        self._dataloader = self._setup_data(cfg.dataset, cfg.shuffle, cfg.batch_size, "torchtune_b200.data.padded_collate_dpo", ckpt.get(training.DATALOADER_KEY) if self._resume_from_checkpoint else None)
        self._val_dataloader = None
        self._run_val_every_n_steps = None
        self._steps_per_epoch = len(self._dataloader) // self._gradient_accumulation_steps
        if self.max_steps_per_epoch is not None and self.max_steps_per_epoch < self._steps_per_epoch:
            self._steps_per_epoch = self.max_steps_per_epoch
        self.global_step = self.epochs_run * self._steps_per_epoch
        self.total_training_steps = self.total_epochs * self._steps_per_epoch
        self._lr_scheduler = self._setup_lr_scheduler(cfg.get("lr_scheduler"), self.total_training_steps, self.global_step - 1)
        self._profiler = self._setup_profiler(cfg.get("profiler"))

    def _setup_reference_model(self, cfg: DictConfig) -> nn.Module:
        ref_cfg = cfg.get("ref_checkpointer") or cfg.checkpointer
        ref_ckpt = config.instantiate(ref_cfg, should_load_recipe_state=False).load_checkpoint()
        with training.set_default_dtype(self._dtype), self._device:
            ref = config.instantiate(cfg.model)
        ref.load_state_dict(ref_ckpt[training.MODEL_KEY])
        ref.eval()
        for p in ref.parameters():
            p.requires_grad_(False)
        utils.log_rank_zero(log, "Reference model is initialized.")
        return ref

    def _setup_data(self, cfg_dataset, shuffle, batch_size, collate_fn, loader_state):
        from functools import partial

        from ..datasets import ConcatDataset
        from .dataloading import StatefulDataLoader, StatefulDistributedSampler

        if isinstance(cfg_dataset, config.ListConfig):
            ds = ConcatDataset(datasets=[config.instantiate(c, self._tokenizer) for c in cfg_dataset])
        else:
            ds = config.instantiate(cfg_dataset, self._tokenizer)
        dp_size = self.parallel.dp_size if self.parallel is not None else 1
        dp_rank = self.parallel.dp_rank if self.parallel is not None else 0
        sampler = StatefulDistributedSampler(ds, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle, seed=0)
        pad_id = getattr(self._tokenizer, "pad_id", 0) if self._tokenizer is not None else 0
        loader = StatefulDataLoader(ds, batch_size=batch_size, sampler=sampler, collate_fn=partial(padded_collate_dpo, padding_idx=pad_id, ignore_idx=CROSS_ENTROPY_IGNORE_IDX), drop_last=True)
        if loader_state is not None:
            loader.load_state_dict(loader_state)
        return loader

    # ------------------------------------------------------------------ forward
    def concatenated_forward(self, model: nn.Module, batch) -> Tuple[ChosenRejectedOutputs, torch.Tensor, torch.Tensor]:
        tokens, labels = batch
        tokens, labels = tokens.to(self._device), labels.to(self._device)
        n_chosen = tokens.shape[0] // 2
        with self._activations_ctx:
            logps, mean_logits = sequence_logprobs(model, tokens, labels)
        out = ChosenRejectedOutputs(chosen_logps=logps[:n_chosen], rejected_logps=logps[n_chosen:])
        return out, mean_logits[:n_chosen].mean(), mean_logits[n_chosen:].mean()

    def _reference_forward(self, batch) -> ChosenRejectedOutputs:
        if getattr(self._loss_fn, "is_reference_free", lambda: False)() is True:
            return ChosenRejectedOutputs(None, None)
        with torch.no_grad():
            if self._ref_model is not None:
                return self.concatenated_forward(self._ref_model, batch)[0]
            with disable_adapter(self._model):
                return self.concatenated_forward(self._model, batch)[0]

    # ------------------------------------------------------------------ train
    def train(self) -> None:
        training.cleanup_before_training()
        self._optimizer.zero_grad()
        timer = StepTimer(self._device)
        params = [p for p in self._model.parameters() if p.requires_grad]
        ga = self._gradient_accumulation_steps
        self._profiler.start()
        for curr_epoch in range(self.epochs_run, self.total_epochs):
            self._dataloader.sampler.set_epoch(curr_epoch)
            pbar = tqdm(total=self._steps_per_epoch, disable=not self._is_rank_zero)
            running = {}
            num_tokens = 0
            timer.start()
            for idx, batch in enumerate(self._dataloader):
                if self.max_steps_per_epoch is not None and (idx // ga) == self.max_steps_per_epoch:
                    break
                num_tokens += batch[0].numel()
                policy, chosen_logit, rejected_logit = self.concatenated_forward(self._model, batch)
                reference = self._reference_forward(batch)
                losses, chosen_rewards, rejected_rewards = self._loss_fn(policy, reference)
                loss = losses.mean() / ga
                loss.backward()
                stats = {
                    "loss": loss.detach(),
                    "rewards/chosen": chosen_rewards.mean() / ga,
                    "rewards/rejected": rejected_rewards.mean() / ga,
                    "rewards/accuracies": (chosen_rewards > rejected_rewards).float().mean() / ga,
                    "rewards/margins": (chosen_rewards - rejected_rewards).mean() / ga,
                    "log_probs/chosen": policy.chosen_logps.detach().mean() / ga,
                    "log_probs/rejected": policy.rejected_logps.detach().mean() / ga,
                    "logits/chosen": chosen_logit / ga,
                    "logits/rejected": rejected_logit / ga,
                }
                for k, v in stats.items():
                    running[k] = running.get(k, 0.0) + v.float()

                if (idx + 1) % ga == 0:
                    grad_norm = None
                    if self.parallel is not None:
                        # every rank back-propagated its local mean: average over data-parallel ranks
                        grad_norm = self.parallel.optimizer_step(self._model, self._optimizer, 1.0 / self.parallel.dp_size, self._clip_grad_norm)
                        keys = sorted(running)
                        packed = torch.stack([running[k] for k in keys])
                        self.parallel.all_reduce_sum_(packed)
                        running = {k: v / self.parallel.dp_size for k, v in zip(keys, packed)}
                    else:
                        if self._clip_grad_norm is not None:
                            grad_norm = torch.nn.utils.clip_grad_norm_(params, max_norm=float(self._clip_grad_norm))
                        self._optimizer.step()
                        self._optimizer.zero_grad(set_to_none=True)
                    if self._lr_scheduler is not None:
                        self._lr_scheduler.step()
                    self.global_step += 1
                    timer.stop()
                    loss_to_log = running["loss"].item()
                    pbar.update(1)
                    pbar.set_description(f"{curr_epoch + 1}|{self.global_step}|Loss: {loss_to_log}")
                    if self.global_step % self._log_every_n_steps == 0 and self._is_rank_zero:
                        log_dict = {k: v.item() for k, v in running.items()}
                        log_dict["lr"] = training.get_lr(self._optimizer)
                        log_dict["tokens_per_second_per_gpu"] = num_tokens / max(timer.elapsed_s, 1e-9)
                        if grad_norm is not None:
                            log_dict["grad_norm"] = float(grad_norm)
                        if self._log_peak_memory_stats:
                            log_dict.update(training.get_memory_stats(device=self._device))
                        self._metric_logger.log_dict(log_dict, step=self.global_step)
                    running = {}
                    num_tokens = 0
                    if self.save_every_n_steps and self.global_step % self.save_every_n_steps == 0 and self.global_step < self.total_training_steps:
                        self.save_checkpoint(epoch=curr_epoch, full_tensors=False)
                    self._profiler.step()
                    timer.start()
            pbar.close()
            self._dataloader.mark_epoch_end()
            self.epochs_run += 1
            if not self.save_every_n_steps:
                self.save_checkpoint(epoch=curr_epoch)
        if self.save_every_n_steps:
            self.save_checkpoint(epoch=self.total_epochs - 1)
        self._profiler.stop()
