"""Supervised fine-tuning engine shared by the single-device and distributed recipes.

The reference implements each recipe as a long stand-alone class
(recipes/full_finetune_single_device.py:124-718,
recipes/full_finetune_distributed.py:53-1169,
recipes/lora_finetune_distributed.py:134-985).  Here the recipe scripts are thin: they
parse the config and drive :class:`SFTTrainer`, which reads the same config keys and
keeps the same observable behaviour — loss normalised by the global number of unmasked
label tokens, ``tokens_per_second_per_gpu`` accounting, checkpoint cadence and resume
semantics — while parallelism is delegated to :mod:`torchtune_b200.parallel`.
"""
from __future__ import annotations

import os
import time
from functools import partial
from typing import Any, Dict, List, Optional, Union

import torch
from torch import nn
from tqdm import tqdm

from .. import config, modules, training, utils
from ..config import DictConfig, ListConfig
from ..config._resolve import get_component_from_path
from ..data import padded_collate_packed, padded_collate_sft
from ..modules.moe import expert_load_imbalance
from ..modules.peft import (
    get_adapter_params,
    get_adapter_state_dict,
    get_lora_module_names,
    get_merged_lora_ckpt,
    set_trainable_params,
    validate_missing_and_unexpected_for_lora,
)
from ..training.memory import CheckpointedLayer
from .dataloading import StatefulDataLoader, StatefulDistributedSampler
from .timing import StepTimer

log = utils.get_logger("DEBUG")



def _restarted_with_checkpoint(cfg: DictConfig) -> bool:
    """Elastic recovery: when torchrun has restarted the workers after a failure (``tune run --max-restarts N``; the restart
    count is exported as ``TORCHELASTIC_RESTART_COUNT``) and the output directory already holds a complete intermediate
    checkpoint, continue from it instead of starting over.  ``resume_after_restart: False`` switches this off."""
    if int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") or 0) <= 0 or not cfg.get("resume_after_restart", True):
        return False
    from pathlib import Path

    from ..training.checkpointing._utils import get_most_recent_checkpoint

    ckpt_cfg = cfg.get("checkpointer")
    out = (ckpt_cfg.get("output_dir") if ckpt_cfg is not None else None) or cfg.get("output_dir")
    recent = get_most_recent_checkpoint(Path(out)) if out else None
    found = recent is not None and ((recent / "recipe_state.pt").exists() or (recent / "metadata.json").exists())
    if found:
        log.info(f"Restart {os.environ['TORCHELASTIC_RESTART_COUNT']} of this job: resuming from {recent}")
    return found


class SFTTrainer:
    """Full / LoRA / QLoRA / DoRA supervised fine-tuning.

    ``distributed=False`` runs on one device; ``distributed=True`` initialises the process
    group and shards the model with the package's own ZeRO-3 sharder
    (:mod:`torchtune_b200.parallel.fsdp`).
    """

    def __init__(self, cfg: DictConfig, *, distributed: bool = False, lora: bool = False) -> None:
        self.cfg = cfg
        self.distributed = distributed
        self.is_lora = lora
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(cfg.get("dtype"), device=self._device)
        if self._dtype == torch.float16:
            raise ValueError("full fp16 training is not supported with this recipe. Please use bf16 or fp32 instead.")
        self.parallel = None
        if distributed:
            from .. import parallel

            self.parallel = parallel.init_from_config(cfg, self._device)
        self.world_size, self.rank = utils.get_world_size_and_rank()
        self._is_rank_zero = self.rank == 0

        self._output_dir = cfg.output_dir
        self._log_every_n_steps = cfg.get("log_every_n_steps", 1)
        self._log_peak_memory_stats = cfg.get("log_peak_memory_stats", False)
        if self._log_peak_memory_stats and self._device.type != "cuda":
            log.info("log_peak_memory_stats was set to True, however, training does not use cuda. Setting log_peak_memory_stats=False.")
            self._log_peak_memory_stats = False

        self._resume_from_checkpoint = cfg.get("resume_from_checkpoint", False) or _restarted_with_checkpoint(cfg)
        self._gradient_accumulation_steps = cfg.get("gradient_accumulation_steps", 1)
        self._optimizer_in_bwd = cfg.get("optimizer_in_bwd", False)
        self._clip_grad_norm = cfg.get("clip_grad_norm", None)
        self._save_adapter_weights_only = cfg.get("save_adapter_weights_only", False)
        if self._optimizer_in_bwd:
            if self._clip_grad_norm is not None:
                raise RuntimeError("Gradient clipping is not supported with optimizer in bwd. Please set clip_grad_norm=None, or optimizer_in_bwd=False.")
            if self._gradient_accumulation_steps > 1:
                raise RuntimeError("Gradient accumulation is not supported with optimizer in bwd. Please set gradient_accumulation_steps=1, or optimizer_in_bwd=False.")

        self._enable_activation_checkpointing = cfg.get("enable_activation_checkpointing", False)
        self._enable_activation_offloading = cfg.get("enable_activation_offloading", False)
        if self._enable_activation_offloading and self._device.type != "cuda":
            raise RuntimeError("enable_activation_offloading should only be True when training on CUDA")

        self.seed = training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode", None))
        self.epochs_run = 0
        self.total_epochs = cfg.epochs
        self.max_steps_per_epoch = cfg.get("max_steps_per_epoch")
        self.global_step = 0
        self.save_every_n_steps = cfg.get("save_every_n_steps")
        self._checkpointer = None
        self._metric_logger = None
        self._profiler = None
        # asynchronous, per-rank sharded intermediate checkpoints (final checkpoints are always full HF-format)
        self._enable_async_checkpointing = cfg.get("enable_async_checkpointing", False)
        self._sharded_checkpointer = None

    # ------------------------------------------------------------------ checkpoint
    def load_checkpoint(self, cfg_checkpointer: DictConfig) -> Dict[str, Any]:
        sharded_resume = False
        if self._enable_async_checkpointing:
            from ..training.checkpointing._utils import get_most_recent_checkpoint

            self._sharded_checkpointer = training.DistributedCheckpointer(checkpoint_dir=cfg_checkpointer.checkpoint_dir, output_dir=cfg_checkpointer.get("output_dir") or self._output_dir)
            recent = get_most_recent_checkpoint(self._sharded_checkpointer.output_dir) if self._resume_from_checkpoint else None
            sharded_resume = recent is not None and os.path.exists(os.path.join(str(recent), "metadata.json"))
        self._checkpointer = config.instantiate(cfg_checkpointer, should_load_recipe_state=self._resume_from_checkpoint and not sharded_resume)
        ckpt = self._checkpointer.load_checkpoint()
        if sharded_resume:
            shard = self._sharded_checkpointer.load_checkpoint()
            self._sharded_opt_state = shard.pop(training.OPT_KEY, None)
            if self.parallel is not None and self.world_size > 1:
                # rank 0's shard carries the replicated weights and the recipe state
                obj = [shard if self._is_rank_zero else None]
                torch.distributed.broadcast_object_list(obj, src=0)
                shard = obj[0]
            ckpt.update(shard)
        if self._resume_from_checkpoint:
            self._update_recipe_state(ckpt)
        return ckpt

    def _update_recipe_state(self, ckpt: Dict[str, Any]) -> None:
        try:
            self.epochs_run = ckpt[training.EPOCHS_KEY]
            if self.seed != ckpt[training.SEED_KEY]:
                import warnings

                warnings.warn(f"Config value for seed does not match the checkpoint value, using the checkpoint value: {ckpt[training.SEED_KEY]}")
                self.seed = ckpt[training.SEED_KEY]
            if self.max_steps_per_epoch != ckpt[training.MAX_STEPS_KEY]:
                import warnings

                warnings.warn(f"Config value for max_steps_per_epoch does not match the checkpoint value, using the checkpoint value: {ckpt[training.MAX_STEPS_KEY]}")
                self.max_steps_per_epoch = ckpt[training.MAX_STEPS_KEY]
            if self.total_epochs != ckpt[training.TOTAL_EPOCHS_KEY]:
                import warnings

                warnings.warn(f"Config value for total_epochs does not match the checkpoint value, using the config value: {self.total_epochs}")
            self._resumed_steps = ckpt.get(training.STEPS_KEY)
        except KeyError as exc:
            raise KeyError("Checkpoint does not contain the required keys needed for updating recipe state. Are you sure you passed in the right recipe checkpoint?") from exc

    # ------------------------------------------------------------------ setup
    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        if self._is_rank_zero:
            self._metric_logger = config.instantiate(cfg.metric_logger)
            self._metric_logger.log_config(cfg)

        ckpt = self.load_checkpoint(cfg.checkpointer)
        self._loss_fn = config.instantiate(cfg.loss)
        self._model = self._setup_model(cfg, ckpt)
        self._tokenizer = config.instantiate(cfg.tokenizer) if cfg.get("tokenizer") is not None else None
        self._optimizer = self._setup_optimizer(cfg.optimizer, ckpt.get(training.OPT_KEY) if self._resume_from_checkpoint else None)

        if hasattr(self._loss_fn, "set_model_output"):
            self._loss_fn.set_model_output(self._model)
        utils.log_rank_zero(log, "Loss is initialized.")

        collate_name = cfg.get("collate_fn", "torchtune_b200.data.padded_collate_sft")
        self._dataloader = self._setup_data(cfg.dataset, cfg.shuffle, cfg.batch_size, collate_name, ckpt.get(training.DATALOADER_KEY) if self._resume_from_checkpoint else None)
        self._val_dataloader = None
        if cfg.get("dataset_val") is not None:
            self._val_dataloader = self._setup_data(cfg.dataset_val, False, cfg.get("batch_size_val", cfg.batch_size), collate_name, None)
        self._run_val_every_n_steps = cfg.get("run_val_every_n_steps")

        self._steps_per_epoch = len(self._dataloader) // self._gradient_accumulation_steps
        if self.max_steps_per_epoch is not None and self.max_steps_per_epoch < self._steps_per_epoch:
            self._steps_per_epoch = self.max_steps_per_epoch
        self.global_step = self.epochs_run * self._steps_per_epoch
        if getattr(self, "_resumed_steps", None):
            self.global_step = self._resumed_steps
        self.total_training_steps = self.total_epochs * self._steps_per_epoch
        self._lr_scheduler = self._setup_lr_scheduler(cfg.get("lr_scheduler"), self.total_training_steps, self.global_step - 1)
        self._profiler = self._setup_profiler(cfg.get("profiler"))
        self.ignore_labels_cache = torch.full((cfg.batch_size, 1), getattr(self._loss_fn, "ignore_index", -100), device=self._device)

    def _setup_profiler(self, cfg_profiler: Optional[DictConfig]):
        from ..training._profiler import DummyProfiler, setup_torch_profiler

        if cfg_profiler is None:
            return DummyProfiler()
        cfg_profiler = DictConfig(config.OmegaConf.to_container(cfg_profiler, resolve=True))
        if cfg_profiler.get("_component_") is None:
            cfg_profiler["_component_"] = "torchtune_b200.training.setup_torch_profiler"
        profiler, profiler_cfg = config.instantiate(cfg_profiler)
        utils.log_rank_zero(log, f" Profiler config after instantiation: {profiler_cfg}")
        self.profiler_profile_memory = profiler_cfg.get("profile_memory", False)
        if profiler_cfg.get("enabled"):
            self.profiler_wait_steps = profiler_cfg["wait_steps"]
            self.profiler_warmup_steps = profiler_cfg["warmup_steps"]
            self.profiler_active_steps = profiler_cfg["active_steps"]
        return profiler

    def _setup_model(self, cfg: DictConfig, ckpt: Dict[str, Any]) -> nn.Module:
        t0 = time.perf_counter()
        # parameters stay resident on every rank (180 GB parts), so the model is built directly on
        # the device; there is no meta-device / deferred-init stage to undo
        # … except under tensor / expert parallelism, where the full model may exceed one GPU: it is built on the meta device
        # and the strategy gives each layer storage (from the checkpoint) right before slicing it
        deferred = (not self.is_lora and self.parallel is not None and not cfg.get("resize_token_embeddings")
                    and (int(cfg.get("tensor_parallel_dim", 1) or 1) > 1 or int(cfg.get("expert_parallel_dim", 1) or 1) > 1))
        # … and for a sharded 4-bit base (QLoRA with `shard_parameters`): the whole base may not fit one GPU either
        sharded = cfg.get("shard_parameters", False) and str(cfg.get("shard_parameters")).lower() not in ("false", "none", "0", "")
        # … and for sharded frozen bases (LoRA / QLoRA with `shard_parameters`) and `shard_parameters: linear`: the whole base may not
        # fit one GPU either, so each rank copies its rows of every weight from the checkpoint straight into its shard
        linear_only = str(cfg.get("shard_parameters", "")).lower() == "linear"
        deferred = deferred or bool(self.parallel is not None and sharded and (self.is_lora or linear_only or cfg.get("shard_parameters_layerwise", False))
                                    and not cfg.get("resize_token_embeddings"))
        with training.set_default_dtype(self._dtype), (torch.device("meta") if deferred else self._device):
            model = config.instantiate(cfg.model)
        if cfg.get("resize_token_embeddings") and self._tokenizer_vocab(cfg) is not None:
            modules.resize_token_embeddings(model, self._tokenizer_vocab(cfg))

        if self.is_lora:
            self._lora_rank = cfg.model.lora_rank
            self._lora_alpha = cfg.model.lora_alpha
            self._lora_attn_modules = list(cfg.model.lora_attn_modules)
            self._apply_lora_to_mlp = cfg.model.get("apply_lora_to_mlp", False)
            self._apply_lora_to_output = cfg.model.get("apply_lora_to_output", False)
            self.adapter_params = get_adapter_params(model)
            set_trainable_params(model, self.adapter_params)

        model = self._transform_model(model, cfg)

        if self._enable_activation_checkpointing:
            ac_mode = cfg.get("ac_mode")
            if ac_mode is not None:
                training.apply_selective_activation_checkpointing(model, ac_mode, cfg.get("ac_option"))
            else:
                training.set_activation_checkpointing(model, auto_wrap_policy={modules.TransformerSelfAttentionLayer, modules.TransformerCrossAttentionLayer})

        base_sd = ckpt[training.MODEL_KEY]
        adapter_sd = ckpt.get(training.ADAPTER_KEY)
        if self.parallel is not None:
            model = self.parallel.shard_model(model, cfg, base_sd, adapter_sd, dtype=self._dtype, strict=not self.is_lora)
        else:
            if self.is_lora:
                base_missing, base_unexpected = model.load_state_dict(base_sd, strict=False)
                lora_missing = lora_unexpected = None
                if adapter_sd is not None:
                    lora_missing, lora_unexpected = model.load_state_dict(adapter_sd, strict=False)
                validate_missing_and_unexpected_for_lora(
                    state_dict_keys=list(model.state_dict().keys()),
                    base_missing=base_missing,
                    base_unexpected=base_unexpected,
                    lora_missing=lora_missing,
                    lora_unexpected=lora_unexpected,
                )
                for m in model.modules():
                    if hasattr(m, "initialize_dora_magnitude") and adapter_sd is None:
                        m.initialize_dora_magnitude()
            else:
                model.load_state_dict(base_sd)
            training.validate_expected_param_dtype(
                ((n, p) for n, p in model.named_parameters() if p.requires_grad or not self.is_lora), dtype=self._dtype
            )
        self._activations_ctx = training.get_act_offloading_ctx_manager(model, self._enable_activation_offloading)
        utils.log_rank_zero(log, f"Model is initialized with precision {self._dtype} in {time.perf_counter() - t0:.2f} secs.")
        if self._device.type == "cuda" and self._is_rank_zero:
            training.log_memory_stats(training.get_memory_stats(self._device))
        return model

    def _transform_model(self, model: nn.Module, cfg: DictConfig) -> nn.Module:
        """Hook for engines that rewrite modules before weights are loaded (QAT, fp8)."""
        if cfg.get("enable_fp8_training", False):
            model = training.convert_to_float8_training(model, cfg.get("fp8_recipe_name"))
        return model

    def _before_batch(self, idx: int) -> None:
        """Hook called before every micro-batch."""

    def _after_step(self) -> None:
        """Hook called after every optimizer step."""

    def _tokenizer_vocab(self, cfg) -> Optional[int]:
        tok = getattr(self, "_tokenizer", None)
        return getattr(tok, "vocab_size", None) if tok is not None else None

    def _setup_optimizer(self, cfg_optimizer: DictConfig, opt_state: Optional[Dict[str, Any]]):
        if self._optimizer_in_bwd:
            optim_dict = {p: config.instantiate(cfg_optimizer, [p]) for p in self._model.parameters() if p.requires_grad}
            training.register_optim_in_bwd_hooks(self._model, optim_dict)
            self._optim_ckpt_wrapper = training.create_optim_in_bwd_wrapper(self._model, optim_dict)
            if opt_state is not None:
                self._optim_ckpt_wrapper.load_state_dict(opt_state)
            utils.log_rank_zero(log, "In-backward optimizers are set up.")
            return None
        sharded_state = getattr(self, "_sharded_opt_state", None)
        if sharded_state is not None:
            opt_state = None
        if self.parallel is not None:
            optimizer = self.parallel.build_optimizer(self._model, cfg_optimizer, opt_state)
            if sharded_state is not None:
                optimizer.load_state_dict(sharded_state)
        else:
            optimizer = config.instantiate(cfg_optimizer, [p for p in self._model.parameters() if p.requires_grad])
            if sharded_state is not None:
                optimizer.load_state_dict(sharded_state)
            elif opt_state is not None:
                optimizer.load_state_dict(opt_state)
        utils.log_rank_zero(log, "Optimizer is initialized.")
        return optimizer

    def _setup_lr_scheduler(self, cfg_lr: Optional[DictConfig], num_training_steps: int, last_epoch: int):
        if cfg_lr is None:
            utils.log_rank_zero(log, "No learning rate scheduler configured. Using constant learning rate.")
            return None
        target = self._optimizer
        if self._optimizer_in_bwd:
            target = next(iter(self._optim_ckpt_wrapper.optim_map.values()))
        if target is None or not isinstance(target, torch.optim.Optimizer):
            target = getattr(target, "torch_optimizer", target)
        sched = config.instantiate(cfg_lr, target, num_training_steps=num_training_steps, last_epoch=last_epoch)
        if self._optimizer_in_bwd:
            self._optim_ckpt_wrapper.set_lr_scheduler(sched)
        utils.log_rank_zero(log, "Learning rate scheduler is initialized.")
        return sched

    def _setup_data(self, cfg_dataset, shuffle: bool, batch_size: int, collate_fn: str, loader_state: Optional[Dict[str, Any]]):
        from ..datasets import ConcatDataset

        if isinstance(cfg_dataset, ListConfig):
            parts = [config.instantiate(c, self._tokenizer) for c in cfg_dataset]
            ds = ConcatDataset(datasets=parts)
            packed = getattr(ds, "packed", False)
        else:
            ds = config.instantiate(cfg_dataset, self._tokenizer)
            packed = cfg_dataset.get("packed", False) or "seq_lens" in _peek(ds)
        if "left_pad_sequence" in collate_fn:
            raise RuntimeError("left_pad_sequence collator is only for inference.")
        collate = get_component_from_path(collate_fn)
        dp_size = self.parallel.dp_size if self.parallel is not None else 1
        dp_rank = self.parallel.dp_rank if self.parallel is not None else 0
        sampler = StatefulDistributedSampler(ds, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle, seed=0)
        pad_multiple = self.parallel.min_seq_len_divisor if self.parallel is not None else 1
        pad_id = getattr(self._tokenizer, "pad_id", 0) if self._tokenizer is not None else 0
        ignore = getattr(self._loss_fn, "ignore_index", -100)
        if packed:
            fn = padded_collate_packed
        else:
            fn = partial(collate, padding_idx=pad_id, ignore_idx=ignore, pad_to_multiple_of=pad_multiple)
        loader = StatefulDataLoader(ds, batch_size=batch_size, sampler=sampler, collate_fn=fn, drop_last=True, pin_memory=self._device.type == "cuda")
        if loader_state is not None:
            loader.load_state_dict(loader_state)
        return loader

    # ------------------------------------------------------------------ checkpoint save
    def save_checkpoint(self, *, epoch: int, full_tensors: bool = True) -> None:
        intermediate = self.global_step < self.total_training_steps if self.save_every_n_steps else epoch + 1 < self.total_epochs
        t0 = time.perf_counter()
        if intermediate and self._sharded_checkpointer is not None and not self._optimizer_in_bwd:
            self._save_sharded(epoch)
            return
        if self.parallel is not None:
            model_sd = self.parallel.gather_full_state_dict(self._model)
            opt_sd = self.parallel.gather_optimizer_state_dict(self._model, self._optimizer) if intermediate else None
        else:
            model_sd = {k: v.detach().cpu() if not self.is_lora else v.detach() for k, v in self._model.state_dict().items()}
            opt_sd = None
            if intermediate:
                opt_sd = self._optim_ckpt_wrapper.state_dict() if self._optimizer_in_bwd else self._optimizer.state_dict()
        if self._is_rank_zero:
            ckpt: Dict[str, Any] = {}
            if intermediate:
                ckpt.update(
                    {
                        training.OPT_KEY: opt_sd,
                        training.SEED_KEY: self.seed,
                        training.EPOCHS_KEY: self.epochs_run,
                        training.TOTAL_EPOCHS_KEY: self.total_epochs,
                        training.MAX_STEPS_KEY: self.max_steps_per_epoch,
                        training.STEPS_KEY: self.global_step,
                        training.DATALOADER_KEY: self._dataloader.state_dict(),
                    }
                )
            if self.is_lora:
                adapter = get_adapter_state_dict(model_sd)
                ckpt[training.ADAPTER_KEY] = adapter
                merged = get_merged_lora_ckpt({k: v.clone() if k.endswith(".weight") and "lora" not in k else v for k, v in model_sd.items()}, rank=self._lora_rank, alpha=self._lora_alpha)
                ckpt[training.MODEL_KEY] = {k: v.cpu() for k, v in merged.items()}
                ckpt[training.ADAPTER_CONFIG] = {
                    "r": self._lora_rank,
                    "lora_alpha": self._lora_alpha,
                    "target_modules": get_lora_module_names(self._lora_attn_modules, self._apply_lora_to_mlp, self._apply_lora_to_output),
                    "peft_type": "LORA",
                }
            else:
                ckpt[training.MODEL_KEY] = model_sd
            self._checkpointer.save_checkpoint(
                ckpt,
                epoch=epoch,
                intermediate_checkpoint=intermediate,
                adapter_only=self._save_adapter_weights_only and self.is_lora,
                step=self.global_step if self.save_every_n_steps else None,
                dir_prefix="step" if self.save_every_n_steps else "epoch",
            )
            log.info(f"Saving checkpoint took {time.perf_counter() - t0:.2f} secs")
        if self.parallel is not None:
            self.parallel.barrier()

    def _save_sharded(self, epoch: int) -> None:
        """Intermediate checkpoint: every rank snapshots its own optimizer shard (rank 0 also the resident weights
        and the recipe state) to host memory and a writer thread persists it while training continues."""
        state: Dict[str, Any] = {training.OPT_KEY: self._optimizer.state_dict()}
        if self._is_rank_zero:
            sd = self._model.state_dict()
            if self.is_lora:
                sd = get_adapter_state_dict(sd)
            state[training.ADAPTER_KEY if self.is_lora else training.MODEL_KEY] = sd
            state.update(
                {
                    training.SEED_KEY: self.seed,
                    training.EPOCHS_KEY: self.epochs_run,
                    training.TOTAL_EPOCHS_KEY: self.total_epochs,
                    training.MAX_STEPS_KEY: self.max_steps_per_epoch,
                    training.STEPS_KEY: self.global_step,
                    training.DATALOADER_KEY: self._dataloader.state_dict(),
                }
            )
        self._sharded_checkpointer.save_checkpoint(state, epoch=epoch, save_async=True, step=self.global_step if self.save_every_n_steps else None, dir_prefix="step" if self.save_every_n_steps else "epoch")

    # ------------------------------------------------------------------ train
    def _loss_step(self, batch: Dict[str, Any]):
        """Returns ``(loss_sum, n_valid)`` for one micro-batch."""
        cp = getattr(self._model, "_cp", None)
        if cp is not None:  # context parallel: this rank's slice of every sequence (the mask still describes whole sequences)
            batch = cp.shard_batch(batch)
        labels = batch.pop("labels")
        if hasattr(self._model, "shard_rows"):  # tensor parallel: the loss runs on this rank's token rows
            labels = self._model.shard_rows(labels)
        with self._activations_ctx:
            outputs = self._model(**batch)
        if hasattr(self._loss_fn, "compute_sum"):
            if isinstance(outputs, list):  # hidden-state taps: the last entry is the model output
                outputs = outputs[-1]
            return self._loss_fn.compute_sum(outputs, labels)
        n_valid = (labels != getattr(self._loss_fn, "ignore_index", -100)).sum()
        if isinstance(outputs, list):
            loss = self._loss_fn(outputs, labels)
        else:
            loss = self._loss_fn(outputs.reshape(-1, outputs.size(-1)), labels.reshape(-1))
        return loss * n_valid, n_valid

    def _add_aux_sum(self, name: str, value: torch.Tensor) -> None:
        """Accumulate a token-summed auxiliary metric (logged as ``sum / num_tokens`` each step)."""
        sums = self.__dict__.setdefault("_aux_sums", {})
        sums[name] = sums.get(name, 0.0) + value.detach().float()

    def _reduce_aux_sums(self, num_tokens: torch.Tensor) -> Dict[str, float]:
        sums = self.__dict__.get("_aux_sums") or {}
        if not sums:
            return {}
        keys = sorted(sums)
        packed = torch.stack([sums[k] for k in keys])
        if self.parallel is not None:
            self.parallel.all_reduce_sum_(packed)
        out = {k: (v / num_tokens).item() for k, v in zip(keys, packed)}
        self._aux_sums = {}
        return out

    @torch.no_grad()
    def validate(self) -> Dict[str, float]:
        self._model.eval()
        total = torch.zeros((), device=self._device)
        count = torch.zeros((), device=self._device)
        for batch in self._val_dataloader:
            utils.batch_to_device(batch, self._device)
            s, n = self._loss_step(batch)
            total += s.float()
            count += n
        if self.parallel is not None:
            self.parallel.all_reduce_sum_(total, count)
        self._model.train()
        val = (total / count.clamp_min(1)).item()
        if self._is_rank_zero:
            self._metric_logger.log_dict({"val_loss": val}, step=self.global_step)
        return {"val_loss": val}

    def train(self) -> None:
        training.cleanup_before_training()
        if self._optimizer is not None:
            self._optimizer.zero_grad()
        timer = StepTimer(self._device)
        running_loss = torch.zeros((), device=self._device, dtype=torch.float32)
        num_tokens = torch.zeros((), device=self._device, dtype=torch.float32)
        self._profiler.start()
        non_dp = self.parallel.non_data_parallel_size if self.parallel is not None else 1
        params = [p for p in self._model.parameters() if p.requires_grad]

        for curr_epoch in range(self.epochs_run, self.total_epochs):
            self._dataloader.sampler.set_epoch(curr_epoch)
            pbar = tqdm(total=self._steps_per_epoch, disable=not self._is_rank_zero)
            timer.start()
            for idx, batch in enumerate(self._dataloader):
                if self.max_steps_per_epoch is not None and (idx // self._gradient_accumulation_steps) == self.max_steps_per_epoch:
                    break
                self._before_batch(idx)
                utils.batch_to_device(batch, self._device)
                loss_sum, n_valid = self._loss_step(batch)
                running_loss += loss_sum.detach().float()
                num_tokens += n_valid
                if self._optimizer_in_bwd:
                    # normalise before backward: the update happens inside it
                    if self.parallel is not None:
                        self.parallel.all_reduce_sum_(num_tokens)
                    (loss_sum * (self.world_size / num_tokens)).backward()
                else:
                    last_micro = (idx + 1) % self._gradient_accumulation_steps == 0
                    counted = False
                    if last_micro and self.parallel is not None and getattr(self.parallel, "wants_backward_overlap", lambda _o: False)(self._optimizer):
                        # the global token count is final before this backward: the data-parallel engine consumes each layer's
                        # gradients (reduce, update, broadcast) while backward is still running on the earlier layers
                        self.parallel.all_reduce_sum_(num_tokens, running_loss)
                        counted = True
                        self.parallel.arm_backward_overlap(self._optimizer, 1.0 / num_tokens, self._clip_grad_norm)
                    loss_sum.backward()

                if (idx + 1) % self._gradient_accumulation_steps == 0:
                    grad_norm = None
                    if not self._optimizer_in_bwd:
                        if self.parallel is not None:
                            if not counted:
                                self.parallel.all_reduce_sum_(num_tokens, running_loss)
                            grad_norm = self.parallel.optimizer_step(self._model, self._optimizer, 1.0 / num_tokens, self._clip_grad_norm)
                        else:
                            training.scale_grads_(params, 1.0 / num_tokens)
                            if self._clip_grad_norm is not None:
                                grad_norm = torch.nn.utils.clip_grad_norm_(params, max_norm=float(self._clip_grad_norm))
                            self._optimizer.step()
                            self._optimizer.zero_grad(set_to_none=True)
                    elif self.parallel is not None:
                        self.parallel.all_reduce_sum_(running_loss)
                    if self._lr_scheduler is not None:
                        self._lr_scheduler.step()
                    self.global_step += 1
                    self._after_step()

                    timer.stop()
                    aux = self._reduce_aux_sums(num_tokens)
                    loss_to_log = (running_loss / num_tokens).item()
                    pbar.update(1)
                    pbar.set_description(f"{curr_epoch + 1}|{self.global_step}|Loss: {loss_to_log}")
                    if self.global_step % self._log_every_n_steps == 0 and self._is_rank_zero:
                        step_time = timer.elapsed_s
                        lr = training.get_lr(self._optimizer if not self._optimizer_in_bwd else self._optim_ckpt_wrapper)
                        log_dict = {
                            "loss": loss_to_log,
                            "lr": lr,
                            "tokens_per_second_per_gpu": (num_tokens.item() / non_dp) / (step_time * self.world_size),
                        }
                        if self._log_peak_memory_stats:
                            log_dict.update(training.get_memory_stats(device=self._device))
                        if grad_norm is not None:
                            log_dict["grad_norm"] = float(grad_norm)
                        log_dict.update(aux)
                        imbalance = expert_load_imbalance(self._model)
                        if imbalance is not None:
                            log_dict["moe_load_imbalance"] = float(imbalance)
                        self._metric_logger.log_dict(log_dict, step=self.global_step)
                    running_loss.zero_()
                    num_tokens.zero_()

                    if self.save_every_n_steps and self.global_step % self.save_every_n_steps == 0 and self.global_step < self.total_training_steps:
                        self.save_checkpoint(epoch=curr_epoch, full_tensors=False)
                    if self._run_val_every_n_steps and self._val_dataloader is not None and self.global_step % self._run_val_every_n_steps == 0:
                        pbar.refresh()
                        self.validate()
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

    def cleanup(self) -> None:
        if self._sharded_checkpointer is not None:
            self._sharded_checkpointer.wait()
        if self._is_rank_zero and self._metric_logger is not None:
            self._metric_logger.close()
        if self.parallel is not None:
            self.parallel.shutdown()


def _peek(ds) -> Dict[str, Any]:
    try:
        return ds[0] if len(ds) else {}
    except Exception:
        return {}
