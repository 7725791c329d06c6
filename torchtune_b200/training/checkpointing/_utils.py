"""Checkpoint constants and filesystem helpers (parity: torchtune/training/checkpointing/_utils.py:29-752)."""
from __future__ import annotations

import json
import os
import re
import shutil
import string
from enum import Enum
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Union
from warnings import warn

import torch
from safetensors import safe_open

from ...utils import get_logger

logger = get_logger("DEBUG")

ADAPTER_CONFIG = "adapter_config"
ADAPTER_CONFIG_FNAME = "adapter_config"
ADAPTER_MODEL_FNAME = "adapter_model"
SAFETENSOR_INDEX_FNAME = "model.safetensors.index.json"
TORCH_INDEX_FNAME = "pytorch_model.bin.index.json"
SHARD_FNAME = "model-{cpt_idx}-of-{num_shards}"
RECIPE_STATE_DIRNAME = "recipe_state"
REPO_ID_FNAME = "original_repo_id"
SUFFIXES_TO_NOT_COPY = [
    ".pt",
    ".pth",
    ".bin",
    ".safetensors",
    SAFETENSOR_INDEX_FNAME,
    TORCH_INDEX_FNAME,
    ADAPTER_CONFIG_FNAME,
    ADAPTER_MODEL_FNAME,
]

# keys of the dict exchanged between recipes and checkpointers
ADAPTER_KEY = "adapter"
EPOCHS_KEY = "epochs_run"
MAX_STEPS_KEY = "max_steps_per_epoch"
MODEL_KEY = "model"
OPT_KEY = "optimizer"
SEED_KEY = "seed"
TOTAL_EPOCHS_KEY = "total_epochs"
STEPS_KEY = "steps_run"
RNG_KEY = "rng_state"
DATALOADER_KEY = "dataloader"
VAL_DATALOADER_KEY = "val_dataloader"


class ModelType(Enum):
    """Architecture tag selecting the weight-conversion rules of a checkpointer."""

    GEMMA = "gemma"
    GEMMA2 = "gemma2"
    LLAMA2 = "llama2"
    LLAMA3 = "llama3"
    LLAMA3_2 = "llama3_2"
    LLAMA3_VISION = "llama3_vision"
    LLAMA4 = "llama4"
    MISTRAL = "mistral"
    PHI3_MINI = "phi3_mini"
    PHI4 = "phi4"
    REWARD = "reward"
    QWEN2 = "qwen2"
    CLIP_TEXT = "clip_text"
    T5_ENCODER = "t5_encoder"
    QWEN3 = "qwen3"


class FormattedCheckpointFiles:
    """Compact description of ``file_{i}_of_{n}`` shard lists: a two-placeholder format
    string and the zero-padded index of the last shard (a *string*, e.g. ``"00004"``)."""

    def __init__(self, filename_format: str, max_filename: str):
        self.filename_format = filename_format
        self.max_filename = max_filename
        fields = [f for _, f, _, _ in string.Formatter().parse(filename_format) if f is not None]
        if len(fields) != 2:
            raise ValueError("Filename format string must have exactly two placeholders, e.g. 'file_{i}_of_{n_files}.pth'")

    @classmethod
    def from_dict(cls, d: dict) -> "FormattedCheckpointFiles":
        if "filename_format" not in d or "max_filename" not in d:
            raise ValueError("Must pass 'filename_format' and 'max_filename' keys to generate checkpoint filenames")
        if not isinstance(d["max_filename"], str):
            raise ValueError(f"`max_filename` must be a string, but found {type(d['max_filename'])} instead.")
        return cls(d["filename_format"], d["max_filename"])

    def build_checkpoint_filenames(self) -> List[str]:
        width, count = len(self.max_filename), int(self.max_filename)
        return [self.filename_format.format(str(i).zfill(width), self.max_filename) for i in range(1, count + 1)]


def get_path(input_dir: Union[Path, str], filename: str, missing_ok: bool = False) -> Path:
    input_dir = Path(input_dir)
    if not input_dir.is_dir():
        raise ValueError(f"{input_dir} is not a valid directory.")
    path = input_dir / filename
    if not missing_ok and not path.is_file():
        raise ValueError(f"No file with name: {filename} found in {input_dir}.")
    return path


def safe_torch_load(checkpoint_path: Union[Path, str], weights_only: bool = True, mmap: bool = True) -> Dict[str, Any]:
    """Load ``.safetensors`` (zero-copy) or a pickled torch file (memory-mapped, weights only)."""
    path = str(checkpoint_path)
    try:
        if path.endswith(".safetensors"):
            out = {}
            with safe_open(path, framework="pt", device="cpu") as f:
                for k in f.keys():
                    out[k] = f.get_tensor(k)
            return out
        return torch.load(path, map_location="cpu", mmap=mmap, weights_only=weights_only)
    except Exception as exc:
        raise ValueError(f"Unable to load checkpoint from {checkpoint_path}. ") from exc


def update_state_dict_for_classifier(state_dict: Dict[str, torch.Tensor], model_named_parameters: Iterable, force_override: bool = False) -> None:
    """When loading a language-model checkpoint into a classifier, keep the freshly
    initialised ``output.weight`` of the model if the row counts differ (or always with
    ``force_override``); any ``output.bias`` in the checkpoint is dropped."""
    named = dict(model_named_parameters)
    if "output.weight" not in state_dict:
        raise AssertionError("Expected output.weight in state_dict, but it wasn't found.")
    if "output.weight" not in named:
        raise AssertionError("Expected output.weight in model_named_parameters, but it wasn't found.")
    if "output.bias" in state_dict:
        warn("Found output.bias in state dict - this will not be used!")
        state_dict.pop("output.bias")
    if force_override or state_dict["output.weight"].shape[0] != named["output.weight"].shape[0]:
        state_dict["output.weight"] = named["output.weight"]


_CKPT_DIR = re.compile(r"^(epoch|step)_(\d+)$")


def get_all_checkpoints_in_dir(dir: Path, *, pattern: str = r"^(epoch|step)_(\d+)") -> List[Path]:
    rx = re.compile(pattern)
    if not Path(dir).is_dir():
        return []
    # ``<name>.partial`` is a checkpoint whose writers had not all finished when the job stopped: never a candidate
    return [p for p in Path(dir).iterdir() if p.is_dir() and rx.match(p.name) and not p.name.endswith(".partial")]


def _ckpt_order(p: Path):
    m = re.match(r"^(epoch|step)_(\d+)", p.name)
    return (int(m.group(2)), p.stat().st_mtime)


def get_most_recent_checkpoint(dir: Path) -> Optional[Path]:
    """Newest non-empty ``epoch_N`` / ``step_N`` directory under ``dir``."""
    candidates = [p for p in get_all_checkpoints_in_dir(Path(dir)) if any(p.iterdir())]
    return max(candidates, key=_ckpt_order) if candidates else None


def get_largest_iter_folder(dir: Union[str, Path], pattern: str = r"^epoch_(\d+)") -> Optional[str]:
    rx = re.compile(pattern)
    best, best_n = None, -1
    for p in Path(dir).iterdir():
        m = rx.match(p.name)
        if m and int(m.group(1)) > best_n:
            best, best_n = p.name, int(m.group(1))
    return best


def prune_surplus_checkpoints(checkpoints: List[Path], keep_last_n_checkpoints: int = 1) -> None:
    if keep_last_n_checkpoints < 1:
        raise ValueError("keep_last_n_checkpoints must be greater than or equal to 1")
    ordered = sorted(checkpoints, key=_ckpt_order)
    for stale in ordered[: max(0, len(ordered) - keep_last_n_checkpoints)]:
        shutil.rmtree(stale, ignore_errors=True)


def check_outdir_not_in_ckptdir(ckpt_dir: Union[str, Path], out_dir: Union[str, Path]) -> bool:
    ckpt, out = Path(ckpt_dir).resolve(), Path(out_dir).resolve()
    if out == ckpt or ckpt in out.parents:
        raise ValueError(
            f"The output directory cannot be the same as or a subdirectory of the checkpoint directory. Found checkpoint_dir={ckpt_dir} and output_dir={out_dir}."
        )
    return True


def copy_files(input_dir: Union[str, Path], output_dir: Union[str, Path], *, ignore_suffixes: Optional[Sequence[str]] = None, max_file_size_mb: int = 100) -> None:
    """Mirror the small non-weight files (tokenizer, config.json, …) of ``input_dir``."""
    limit = max_file_size_mb * 1024 * 1024
    for root, dirs, files in os.walk(input_dir):
        dirs[:] = [d for d in dirs if not d.startswith(".")]
        dest = Path(output_dir) / os.path.relpath(root, input_dir)
        dest.mkdir(parents=True, exist_ok=True)
        for name in files:
            if name.startswith(".") or (ignore_suffixes and any(name.endswith(s) for s in ignore_suffixes)):
                continue
            src = Path(root) / name
            if src.stat().st_size > limit:
                print(f"Skipping copying {src} to {output_dir} as it exceeds the size limit of {max_file_size_mb} MiB.")
                continue
            if not (dest / name).exists():
                shutil.copy2(src, dest / name)


def get_recipe_checkpoint_path(output_dir, checkpoint_dir, recipe_checkpoint: Optional[str] = None, should_load_recipe_state: bool = False) -> Optional[Path]:
    if not should_load_recipe_state:
        return None
    path = Path(output_dir) / recipe_checkpoint if recipe_checkpoint else Path(checkpoint_dir) / "recipe_state.pt"
    if not path.exists():
        raise ValueError(f"If `should_load_recipe_state=True`, recipe_checkpoint file must be provided. Could not find it at {path}.")
    return path


def get_adapter_checkpoint_path(output_dir, adapter_checkpoint: Optional[str] = None, should_load_recipe_state: bool = False, pattern: str = r"^epoch_(\d+)") -> Optional[Path]:
    if not should_load_recipe_state:
        return None
    if adapter_checkpoint:
        path = Path(output_dir) / adapter_checkpoint
    else:
        folder = get_largest_iter_folder(output_dir, pattern=pattern)
        if folder is None:
            return None
        path = Path(output_dir) / folder / "adapter_model.pt"
    return path if path.exists() else None


def get_model_checkpoint_path(
    checkpoint_files: Union[List[str], Dict[str, str], FormattedCheckpointFiles],
    checkpoint_dir: Union[str, Path],
    output_dir: Union[str, Path],
    should_load_recipe_state: bool,
    has_adapter_checkpoint: bool,
) -> List[Path]:
    """Resolve the weight files to read.  When resuming a full-model run (no adapter) the
    files come from the resumed ``output_dir`` checkpoint instead of ``checkpoint_dir``."""
    if isinstance(checkpoint_files, dict) or hasattr(checkpoint_files, "keys"):
        checkpoint_files = FormattedCheckpointFiles.from_dict(dict(checkpoint_files))
    if isinstance(checkpoint_files, FormattedCheckpointFiles):
        names = checkpoint_files.build_checkpoint_filenames()
    else:
        names = list(checkpoint_files)
    base = Path(output_dir) if (should_load_recipe_state and not has_adapter_checkpoint) else Path(checkpoint_dir)
    if should_load_recipe_state and not has_adapter_checkpoint:
        # a resumed directory holds whatever shards the previous save produced
        produced = sorted(p.name for p in base.glob("model-*-of-*.safetensors")) or sorted(p.name for p in base.glob("model-*-of-*.bin"))
        if produced:
            names = produced
    return sorted(get_path(base, n) for n in names)


def shard_state_dict(state_dict: Dict[str, torch.Tensor], max_shard_size: int) -> List[Dict[str, torch.Tensor]]:
    """Greedy split in key order so that no shard exceeds ``max_shard_size`` bytes."""
    shards: List[Dict[str, torch.Tensor]] = [{}]
    used = 0
    for k, v in state_dict.items():
        n = v.numel() * v.element_size()
        if shards[-1] and used + n > max_shard_size:
            shards.append({})
            used = 0
        shards[-1][k] = v
        used += n
    return shards


def parse_size(size: Union[int, str]) -> int:
    if isinstance(size, int):
        return size
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([KMGT]i?B)\s*", size, re.I)
    if not m:
        raise ValueError(f"cannot parse size '{size}'")
    unit = m.group(2).upper()
    power = "KMGT".index(unit[0]) + 1
    base = 1024 if "I" in unit else 1000
    return int(float(m.group(1)) * base**power)
