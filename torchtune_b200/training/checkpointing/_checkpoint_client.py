"""Recipe-facing checkpoint façade (parity: torchtune/training/checkpointing/_checkpoint_client.py:36-640).

``CheckpointClient`` hides which checkpointer is used: full-format checkpoints (HF / Meta / native files, with LoRA merged
and adapter files written) go through the configured checkpointer on rank 0; with ``enable_async_checkpointing`` intermediate
checkpoints go through :class:`DistributedCheckpointer` (per-rank shards written by a background thread).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from ... import config, utils
from . import _utils as K
from ._sharded import DistributedCheckpointer

log = utils.get_logger("DEBUG")


@dataclass
class TrainingProgress:
    """What a run needs, besides weights and optimizer state, to continue where it stopped."""

    seed: int
    epochs_run: int
    total_epochs: int
    max_steps_per_epoch: int
    steps_run: Optional[int] = None
    total_training_steps: Optional[int] = None
    dataloader_state_dict: Optional[Dict[str, Any]] = None
    val_dataloader_state_dict: Optional[Dict[str, Any]] = None

    def state_dict(self) -> Dict[str, object]:
        return {
            K.SEED_KEY: self.seed,
            K.EPOCHS_KEY: self.epochs_run,
            K.TOTAL_EPOCHS_KEY: self.total_epochs,
            K.MAX_STEPS_KEY: self.max_steps_per_epoch,
            K.STEPS_KEY: self.steps_run,
            "total_training_steps": self.total_training_steps,
            K.DATALOADER_KEY: self.dataloader_state_dict,
            K.VAL_DATALOADER_KEY: self.val_dataloader_state_dict,
        }


class CheckpointClient:
    def __init__(self, cfg, checkpointer: Optional[Any] = None, parallel: Optional[Any] = None) -> None:
        self._cfg = cfg
        self._checkpointer = checkpointer
        self._sharded: Optional[DistributedCheckpointer] = None
        self._parallel = parallel
        self._resume_from_checkpoint = cfg.get("resume_from_checkpoint", False)
        self._enable_async_checkpointing = cfg.get("enable_async_checkpointing", False)
        self._optimizer_in_bwd = cfg.get("optimizer_in_bwd", False)
        self._device = utils.get_device(device=cfg.get("device"))
        _, self._rank = utils.get_world_size_and_rank()
        self._is_rank_zero = self._rank == 0

    # ------------------------------------------------------------------ checkpointers
    def _get_checkpointer(self):
        if self._checkpointer is None:
            load_recipe_state = False if self._enable_async_checkpointing else self._resume_from_checkpoint
            self._checkpointer = config.instantiate(self._cfg.checkpointer, should_load_recipe_state=load_recipe_state)
        return self._checkpointer

    def _get_sharded_checkpointer(self) -> DistributedCheckpointer:
        if self._sharded is None:
            ck = self._get_checkpointer()
            self._sharded = DistributedCheckpointer(checkpoint_dir=str(ck._checkpoint_dir), output_dir=str(ck._output_dir))
        return self._sharded

    # ------------------------------------------------------------------ save
    def save_checkpoint(self, model: torch.nn.Module, optimizer: Any, training_progress: TrainingProgress, epoch: int, adapter_config: Optional[Dict[str, Any]] = None,
                        adapter_only: bool = False, single_device: bool = False, *, full_tensors: bool = True, dir_prefix: str = "epoch") -> None:
        tp = training_progress
        if tp.steps_run is not None and tp.total_training_steps is not None:
            intermediate = tp.steps_run < tp.total_training_steps
        else:
            intermediate = epoch + 1 < tp.total_epochs
        if not full_tensors and self._enable_async_checkpointing:
            self._save_async(model, optimizer, tp, epoch, adapter_config, adapter_only, dir_prefix)
        else:
            self._save_sync(model, optimizer, tp, epoch, adapter_config, adapter_only, single_device, intermediate, dir_prefix)

    def _save_async(self, model, optimizer, tp: TrainingProgress, epoch, adapter_config, adapter_only, dir_prefix) -> None:
        from ...modules.peft import get_adapter_state_dict

        t0 = time.perf_counter()
        state: Dict[str, Any] = {}
        if optimizer is not None:
            state[K.OPT_KEY] = optimizer.state_dict()
        if self._is_rank_zero:
            sd = model.state_dict()
            if adapter_config is not None:
                state[K.ADAPTER_KEY] = get_adapter_state_dict(sd)
                state[K.ADAPTER_CONFIG] = adapter_config
            if not adapter_only:
                state[K.MODEL_KEY] = sd
            state.update(tp.state_dict())
        self._get_sharded_checkpointer().save_checkpoint(state, epoch=epoch, save_async=True, adapter_only=False, step=tp.steps_run if dir_prefix == "step" else None, dir_prefix=dir_prefix)
        if self._is_rank_zero:
            log.info(f"Asynchronous checkpoint staged in {time.perf_counter() - t0:.2f} secs")

    def _save_sync(self, model, optimizer, tp: TrainingProgress, epoch, adapter_config, adapter_only, single_device, intermediate, dir_prefix) -> None:
        from ...modules.peft import get_adapter_state_dict, get_merged_lora_ckpt

        t0 = time.perf_counter()
        par = None if single_device else self._parallel
        if par is not None:
            model_sd = par.gather_full_state_dict(model)
            opt_sd = par.gather_optimizer_state_dict(model, optimizer) if (intermediate and optimizer is not None) else None
        else:
            model_sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
            opt_sd = optimizer.state_dict() if (intermediate and optimizer is not None) else None
        if self._is_rank_zero:
            ckpt: Dict[str, Any] = {}
            if intermediate:
                ckpt[K.OPT_KEY] = opt_sd
                ckpt.update(tp.state_dict())
            if adapter_config is not None:
                ckpt[K.ADAPTER_KEY] = get_adapter_state_dict(model_sd)
                ckpt[K.ADAPTER_CONFIG] = adapter_config
                if not adapter_only:
                    merged = get_merged_lora_ckpt({k: (v.clone() if k.endswith(".weight") and "lora" not in k else v) for k, v in model_sd.items()}, rank=adapter_config["r"], alpha=adapter_config["lora_alpha"])
                    ckpt[K.MODEL_KEY] = merged
            else:
                ckpt[K.MODEL_KEY] = model_sd
            self._get_checkpointer().save_checkpoint(ckpt, epoch=epoch, intermediate_checkpoint=intermediate, adapter_only=adapter_only, step=tp.steps_run if dir_prefix == "step" else None, dir_prefix=dir_prefix)
            log.info(f"Saving checkpoint took {time.perf_counter() - t0:.2f} secs")
        if par is not None:
            par.barrier()

    # ------------------------------------------------------------------ load
    def load_base_checkpoint(self) -> Dict[str, Any]:
        """The base weights (and, when resuming without sharded checkpoints, the recipe state) from the configured checkpointer."""
        return self._get_checkpointer().load_checkpoint()

    def load_distributed_checkpoint(self, model: torch.nn.Module, optimizer: Any, adapter_config: Optional[Dict[str, Any]] = None, dataloader: Optional[Any] = None, single_device: bool = False) -> Dict[str, Any]:
        """Restore model weights, this rank's optimizer shard and the training progress from the most recent sharded
        checkpoint; returns the progress entries."""
        shard = self._get_sharded_checkpointer().load_checkpoint()
        if optimizer is not None and K.OPT_KEY in shard:
            optimizer.load_state_dict(shard.pop(K.OPT_KEY))
        world, _ = utils.get_world_size_and_rank()
        if world > 1 and torch.distributed.is_initialized():
            obj = [shard if self._is_rank_zero else None]
            torch.distributed.broadcast_object_list(obj, src=0)
            shard = obj[0]
        if K.MODEL_KEY in shard:
            model.load_state_dict(shard.pop(K.MODEL_KEY))
        if K.ADAPTER_KEY in shard:
            model.load_state_dict(shard.pop(K.ADAPTER_KEY), strict=False)
        if dataloader is not None and shard.get(K.DATALOADER_KEY) is not None:
            dataloader.load_state_dict(shard[K.DATALOADER_KEY])
        return shard

    def wait(self) -> None:
        if self._sharded is not None:
            self._sharded.wait()
