"""Checkpoint readers/writers for the HF, Meta and native formats.

Parity: torchtune/training/checkpointing/_checkpointer.py:122-1478.  All three share one
base class that owns the output-directory layout
(``output_dir/{epoch_N|step_N}/…``), recipe state, adapter files, copying of
non-weight files and pruning; subclasses only define how model weights are read and
written.  A checkpoint directory is written under a temporary name and renamed into
place, so an ``epoch_N``/``step_N`` directory that exists is always complete.
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path
from typing import Any, Dict, List, Optional, Protocol, Union

import torch
from safetensors.torch import save_file as save_safetensors_file

from ...models import convert_weights
from ...utils import get_logger
from . import _utils as U
from ._codecs import hf_codec
from ._utils import ModelType

logger = get_logger("DEBUG")


class _CheckpointerInterface(Protocol):
    """``load_checkpoint() -> dict`` with key ``"model"`` (plus recipe-state keys when
    resuming) and ``save_checkpoint(state_dict, epoch, ...)``."""

    def load_checkpoint(self, **kwargs) -> Dict[str, Any]:
        ...

    def save_checkpoint(self, state_dict: Dict[str, Any], **kwargs) -> None:
        ...


class _BaseCheckpointer:
    _PEFT_UNSUPPORTED = (ModelType.PHI3_MINI, ModelType.PHI4, ModelType.LLAMA3_VISION, ModelType.LLAMA4)

    def __init__(
        self,
        checkpoint_dir: str,
        checkpoint_files: Union[List[str], Dict[str, str]],
        model_type: str,
        output_dir: Optional[str],
        adapter_checkpoint: Optional[str],
        recipe_checkpoint: Optional[str],
        resume_from_checkpoint: bool,
        should_load_recipe_state: bool,
        keep_last_n_checkpoints: Optional[int],
    ) -> None:
        self._checkpoint_dir = str(checkpoint_dir)
        self._model_type = ModelType[model_type] if isinstance(model_type, str) else model_type
        self._output_dir = str(output_dir) if output_dir is not None else None
        self._keep_last_n_checkpoints = keep_last_n_checkpoints
        self._should_load_recipe_state = bool(should_load_recipe_state or resume_from_checkpoint)
        if resume_from_checkpoint:
            logger.warning("*resume_from_checkpoint is deprecated. Please use the 'should_load_recipe_state' instead")
        if self._output_dir is None:
            raise ValueError("Output directory not specified. Please specify an output directory to save the checkpoint.")
        U.check_outdir_not_in_ckptdir(ckpt_dir=self._checkpoint_dir, out_dir=self._output_dir)
        Path(self._output_dir).mkdir(parents=True, exist_ok=True)

        self._recipe_checkpoint: Optional[Path] = None
        self._adapter_checkpoint: Optional[Path] = None
        load_from = Path(self._checkpoint_dir)
        if self._should_load_recipe_state:
            if "step" in Path(self._checkpoint_dir).name or "epoch" in Path(self._checkpoint_dir).name:
                load_from = Path(self._checkpoint_dir)
            else:
                recent = U.get_most_recent_checkpoint(Path(self._output_dir))
                if recent is None:
                    raise ValueError("Recipe state cannot be loaded because no checkpoints were found in the output directory.")
                load_from = recent
            self._recipe_checkpoint = load_from / "recipe_state.pt"
            if not self._recipe_checkpoint.exists():
                raise AssertionError(f"recipe_state.pt not found in {load_from}")
            adapter = load_from / (adapter_checkpoint or "adapter_model.pt")
            self._adapter_checkpoint = adapter if adapter.exists() else None
        self._checkpoint_paths = U.get_model_checkpoint_path(
            checkpoint_files=checkpoint_files,
            checkpoint_dir=self._checkpoint_dir,
            output_dir=load_from if self._should_load_recipe_state else self._output_dir,
            should_load_recipe_state=self._should_load_recipe_state,
            has_adapter_checkpoint=self._adapter_checkpoint is not None,
        )

    # ---- hooks ------------------------------------------------------------
    def _read_model(self) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def _write_model(self, model_sd: Dict[str, torch.Tensor], out_dir: Path, max_shard_size: int) -> None:
        raise NotImplementedError

    def _adapter_to_peft(self, adapter_sd: Dict[str, torch.Tensor]) -> Optional[Dict[str, torch.Tensor]]:
        return None

    repo_id: Optional[str] = None

    # ---- public API ---------------------------------------------------------
    def load_checkpoint(self, **kwargs) -> Dict[str, Any]:
        out: Dict[str, Any] = {U.MODEL_KEY: self._read_model()}
        if self._adapter_checkpoint is not None:
            out[U.ADAPTER_KEY] = U.safe_torch_load(self._adapter_checkpoint)
        if self._should_load_recipe_state:
            out.update(U.safe_torch_load(self._recipe_checkpoint, mmap=False, weights_only=False))
        return out

    def save_checkpoint(
        self,
        state_dict: Dict[str, Any],
        epoch: int,
        intermediate_checkpoint: bool = False,
        adapter_only: bool = False,
        *,
        step: Optional[int] = None,
        max_shard_size: Union[int, str] = "5GB",
        dir_prefix: str = "epoch",
    ) -> None:
        if dir_prefix == "step":
            if step is None:
                raise ValueError("step must be given when dir_prefix='step'")
            name, pattern = f"step_{step}", r"^step_(\d+)"
        else:
            name, pattern = f"epoch_{epoch}", r"^epoch_(\d+)"
        final_dir = Path(self._output_dir) / name
        work_dir = Path(self._output_dir) / f".{name}.partial"
        if work_dir.exists():
            shutil.rmtree(work_dir)
        work_dir.mkdir(parents=True)

        if not adapter_only:
            self._write_model(state_dict[U.MODEL_KEY], work_dir, U.parse_size(max_shard_size))
            logger.info(f"Model checkpoint saved to {final_dir}")

        if U.ADAPTER_KEY in state_dict:
            adapter_sd = state_dict[U.ADAPTER_KEY]
            torch.save(adapter_sd, work_dir / f"{U.ADAPTER_MODEL_FNAME}.pt")
            peft = None if self._model_type in self._PEFT_UNSUPPORTED else self._adapter_to_peft(adapter_sd)
            if peft is not None:
                save_safetensors_file({k: v.contiguous() for k, v in peft.items()}, str(work_dir / f"{U.ADAPTER_MODEL_FNAME}.safetensors"), metadata={"format": "pt"})
            elif self._model_type in self._PEFT_UNSUPPORTED:
                logger.warning("Saving adapter weights to PEFT format is not supported for this model type, saving to native format instead")
        elif adapter_only:
            raise ValueError("Adapter checkpoint not found in state_dict. Please ensure that the state_dict contains adapter weights.")

        if U.ADAPTER_CONFIG in state_dict and self._model_type not in (ModelType.PHI3_MINI, ModelType.PHI4, ModelType.LLAMA3_VISION):
            cfg = convert_weights.tune_to_peft_adapter_config(dict(state_dict[U.ADAPTER_CONFIG]), base_model_name_or_path=self.repo_id)
            (work_dir / f"{U.ADAPTER_CONFIG_FNAME}.json").write_text(json.dumps(cfg))

        U.copy_files(self._checkpoint_dir, work_dir, ignore_suffixes=U.SUFFIXES_TO_NOT_COPY)

        if intermediate_checkpoint:
            recipe_state = {k: v for k, v in state_dict.items() if k not in (U.MODEL_KEY, U.ADAPTER_KEY, U.ADAPTER_CONFIG)}
            torch.save(recipe_state, work_dir / "recipe_state.pt")
            logger.info(f"Recipe checkpoint saved to {final_dir / 'recipe_state.pt'}")
        else:
            logger.info("Saving final epoch checkpoint.")

        if final_dir.exists():
            shutil.rmtree(final_dir)
        os.replace(work_dir, final_dir)

        if self._keep_last_n_checkpoints is not None:
            U.prune_surplus_checkpoints(
                U.get_all_checkpoints_in_dir(Path(self._output_dir), pattern=pattern), keep_last_n_checkpoints=self._keep_last_n_checkpoints
            )


def _write_sharded(sd: Dict[str, torch.Tensor], out_dir: Path, max_shard_size: int, safe: bool) -> None:
    """``model-0000i-of-0000n.safetensors`` (or ``.bin``) plus the HF index json."""
    sd = {k: v.detach().cpu().contiguous() for k, v in sd.items()}
    if safe:
        # safetensors refuses aliased storage; tied tensors are cloned
        seen: Dict[int, str] = {}
        for k, v in list(sd.items()):
            ptr = v.untyped_storage().data_ptr()
            if ptr in seen and v.numel():
                sd[k] = v.clone()
            seen[ptr] = k
    shards = U.shard_state_dict(sd, max_shard_size)
    ext = "safetensors" if safe else "bin"
    weight_map: Dict[str, str] = {}
    for i, shard in enumerate(shards, 1):
        fname = U.SHARD_FNAME.format(cpt_idx=str(i).zfill(5), num_shards=str(len(shards)).zfill(5)) + f".{ext}"
        if safe:
            save_safetensors_file(shard, str(out_dir / fname), metadata={"format": "pt"})
        else:
            torch.save(shard, out_dir / fname)
        weight_map.update({k: fname for k in shard})
    if True:  # the index is written even for a single shard so resumes can discover the files
        total = sum(v.numel() * v.element_size() for v in sd.values())
        index = {"metadata": {"total_size": total}, "weight_map": weight_map}
        (out_dir / (U.SAFETENSOR_INDEX_FNAME if safe else U.TORCH_INDEX_FNAME)).write_text(json.dumps(index, indent=2))


class FullModelHFCheckpointer(_BaseCheckpointer):
    """Reads a HF ``transformers`` checkpoint directory (``config.json`` + safetensors /
    ``.bin`` shards), converts to native keys (q/k rows permuted to the interleaved RoPE
    layout) and writes the same format back."""

    def __init__(
        self,
        checkpoint_dir: str,
        checkpoint_files: Union[List[str], Dict[str, str]],
        model_type: str,
        output_dir: Optional[str] = None,
        adapter_checkpoint: Optional[str] = "adapter_model.pt",
        recipe_checkpoint: Optional[str] = "recipe_state.pt",
        resume_from_checkpoint: bool = False,
        safe_serialization: bool = True,
        should_load_recipe_state: bool = False,
        *,
        keep_last_n_checkpoints: Optional[int] = None,
        enable_dcp: bool = False,
    ) -> None:
        super().__init__(checkpoint_dir, checkpoint_files, model_type, output_dir, adapter_checkpoint, recipe_checkpoint, resume_from_checkpoint, should_load_recipe_state, keep_last_n_checkpoints)
        self._safe_serialization = safe_serialization
        self._enable_dcp = enable_dcp  # accepted for config compatibility; files are read directly
        self._config = json.loads((Path(checkpoint_dir) / "config.json").read_text())
        repo = Path(checkpoint_dir) / f"{U.REPO_ID_FNAME}.json"
        self.repo_id = json.loads(repo.read_text()).get("repo_id") if repo.exists() else None
        self._weight_map: Dict[str, str] = {}

    def _read_model(self) -> Dict[str, torch.Tensor]:
        merged: Dict[str, torch.Tensor] = {}
        self._weight_map = {}
        for idx, path in enumerate(self._checkpoint_paths, 1):
            part = U.safe_torch_load(path)
            for k, v in part.items():
                if not isinstance(v, torch.Tensor):
                    raise ValueError(f"Expected all values in the state dict to be torch.Tensor. Found {type(v)} instead.")
                self._weight_map[k] = f"{idx:04}"
            merged.update(part)
        to_native, _ = hf_codec(self._model_type)
        return to_native(merged, self._config)

    def _write_model(self, model_sd, out_dir: Path, max_shard_size: int) -> None:
        _, from_native = hf_codec(self._model_type)
        _write_sharded(from_native(model_sd, self._config), out_dir, max_shard_size, self._safe_serialization)

    def _adapter_to_peft(self, adapter_sd):
        c = self._config.get("text_config", self._config)
        return convert_weights.tune_to_peft_adapter_weights(
            adapter_sd,
            num_heads=c["num_attention_heads"],
            num_kv_heads=c.get("num_key_value_heads", c["num_attention_heads"]),
            dim=c["hidden_size"],
            head_dim=c.get("head_dim", None),
        )


class FullModelMetaCheckpointer(_BaseCheckpointer):
    """Single-file Meta format (``consolidated.00.pth``).  Llama-3.2 checkpoints tie the
    output projection to the embedding, so ``output.weight`` is dropped on load and
    restored on save."""

    def __init__(
        self,
        checkpoint_dir: str,
        checkpoint_files: List[str],
        model_type: str,
        output_dir: Optional[str] = None,
        adapter_checkpoint: Optional[str] = "adapter_model.pt",
        recipe_checkpoint: Optional[str] = "recipe_state.pt",
        resume_from_checkpoint: bool = False,
        should_load_recipe_state: bool = False,
        *,
        keep_last_n_checkpoints: Optional[int] = None,
    ) -> None:
        if len(checkpoint_files) != 1:
            raise ValueError(f"Currently we only support reading from a single checkpoint file. Got {len(checkpoint_files)} files instead.")
        super().__init__(checkpoint_dir, checkpoint_files, model_type, output_dir, adapter_checkpoint, recipe_checkpoint, resume_from_checkpoint, should_load_recipe_state, keep_last_n_checkpoints)

    def _read_model(self):
        sd = U.safe_torch_load(self._checkpoint_paths[0])
        if self._model_type == ModelType.LLAMA3_VISION:
            from ...models.llama3_2_vision._convert_weights import llama3_vision_meta_to_tune

            return llama3_vision_meta_to_tune(sd)
        if self._model_type == ModelType.LLAMA4:
            from ...models.llama4._convert_weights import llama4_meta_to_tune

            return llama4_meta_to_tune(sd)
        out = convert_weights.meta_to_tune(sd)
        if self._model_type == ModelType.LLAMA3_2:
            out.pop("output.weight", None)
        return out

    def _write_model(self, model_sd, out_dir: Path, max_shard_size: int) -> None:
        if self._model_type == ModelType.LLAMA3_VISION:
            from ...models.llama3_2_vision._convert_weights import llama3_vision_tune_to_meta

            sd = llama3_vision_tune_to_meta(model_sd)
        elif self._model_type == ModelType.LLAMA4:
            from ...models.llama4._convert_weights import llama4_tune_to_meta

            sd = llama4_tune_to_meta(model_sd)
        else:
            model_sd = dict(model_sd)
            if self._model_type == ModelType.LLAMA3_2 and "output.weight" not in model_sd:
                model_sd["output.weight"] = model_sd["tok_embeddings.weight"]
            sd = convert_weights.tune_to_meta(model_sd)
        torch.save({k: v.detach().cpu() for k, v in sd.items()}, out_dir / "model-00001-of-00001.bin")


class FullModelTorchTuneCheckpointer(_BaseCheckpointer):
    """Native format: one file whose keys already match the model's ``state_dict``."""

    def __init__(
        self,
        checkpoint_dir: str,
        checkpoint_files: List[str],
        model_type: str,
        output_dir: Optional[str] = None,
        adapter_checkpoint: Optional[str] = "adapter_model.pt",
        recipe_checkpoint: Optional[str] = "recipe_state.pt",
        resume_from_checkpoint: bool = False,
        should_load_recipe_state: bool = False,
        *,
        keep_last_n_checkpoints: Optional[int] = None,
    ) -> None:
        if len(checkpoint_files) != 1:
            raise ValueError(f"Currently we only support reading from a single checkpoint file. Got {len(checkpoint_files)} files instead.")
        super().__init__(checkpoint_dir, checkpoint_files, model_type, output_dir, adapter_checkpoint, recipe_checkpoint, resume_from_checkpoint, should_load_recipe_state, keep_last_n_checkpoints)

    def load_checkpoint(self, weights_only: bool = True, **kwargs) -> Dict[str, Any]:
        self._weights_only = weights_only
        return super().load_checkpoint()

    def _read_model(self):
        return U.safe_torch_load(self._checkpoint_paths[0], weights_only=getattr(self, "_weights_only", True))

    def _write_model(self, model_sd, out_dir: Path, max_shard_size: int) -> None:
        torch.save({k: v.detach().cpu() if isinstance(v, torch.Tensor) else v for k, v in model_sd.items()}, out_dir / "model-00001-of-00001.bin")
