"""Metric loggers (parity: torchtune/training/metric_logging.py:27-647)."""
from __future__ import annotations

import json
import os
import sys
import time
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Protocol, Union

import torch

from ..config import DictConfig, OmegaConf
from ..utils import get_logger, get_world_size_and_rank

Scalar = Union[torch.Tensor, int, float]
log = get_logger("DEBUG")


def save_config(config: DictConfig) -> Path:
    """Write the resolved config to ``<output_dir>/torchtune_config.yaml``."""
    try:
        out_dir = Path(config.output_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        path = out_dir / "torchtune_config.yaml"
        OmegaConf.save(config, path, resolve=True)
        return path
    except Exception as exc:  # logging must never kill a run
        log.warning(f"Error saving config.\nError: \n{exc}.")
        return Path()


def flatten_dict(d: Dict[str, Any], *, sep: str = ".", parent_key: str = "") -> Dict[str, Any]:
    """``{"a": {"b": 1}, "c": 2}`` → ``{"a.b": 1, "c": 2}`` (dictionaries inside lists are left as they are); used to hand a nested
    config to loggers that take flat hyper-parameter tables."""
    out: Dict[str, Any] = {}
    for key, value in d.items():
        name = f"{parent_key}{sep}{key}" if parent_key else key
        if isinstance(value, dict):
            out.update(flatten_dict(value, sep=sep, parent_key=name))
        else:
            out[name] = value
    return out


def _scalar(v: Scalar) -> float:
    return v.item() if isinstance(v, torch.Tensor) else v


class MetricLoggerInterface(Protocol):
    def log(self, name: str, data: Scalar, step: int) -> None: ...

    def log_config(self, config: DictConfig) -> None: ...

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None: ...

    def close(self) -> None: ...


class DiskLogger(MetricLoggerInterface):
    """Appends ``Step N | k:v k:v`` lines (or json lines) to ``log_dir/<filename>``."""

    def __init__(self, log_dir: str, filename: Optional[str] = None, output_fmt: str = "txt", **kwargs):
        if output_fmt not in ("txt", "jsonl"):
            raise ValueError(f"output_fmt must be 'txt' or 'jsonl', got {output_fmt}")
        self.log_dir = Path(log_dir)
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.output_fmt = output_fmt
        if not filename:
            filename = f"log_{int(time.time())}.{output_fmt}"
        self._file_name = self.log_dir / filename
        self._file = open(self._file_name, "a")
        print(f"Writing logs to {self._file_name}")

    def path_to_log_file(self) -> Path:
        return self._file_name

    def log(self, name: str, data: Scalar, step: int) -> None:
        self.log_dict({name: data}, step)

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        if self.output_fmt == "jsonl":
            self._file.write(json.dumps({"step": step, **{k: _scalar(v) for k, v in payload.items()}}) + "\n")
        else:
            self._file.write(f"Step {step} | " + " ".join(f"{k}:{_scalar(v)}" for k, v in payload.items()) + "\n")
        self._file.flush()

    def log_config(self, config: DictConfig) -> None:
        save_config(config)

    def close(self) -> None:
        if not self._file.closed:
            self._file.close()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class StdoutLogger(MetricLoggerInterface):
    def log(self, name: str, data: Scalar, step: int) -> None:
        print(f"Step {step} | {name}:{_scalar(data)}")

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        print(f"Step {step} | " + " ".join(f"{k}:{_scalar(v)}" for k, v in payload.items()))

    def log_config(self, config: DictConfig) -> None:
        save_config(config)

    def close(self) -> None:
        sys.stdout.flush()

    def __del__(self) -> None:
        self.close()


class _RankZeroBackend(MetricLoggerInterface):
    """Shared plumbing of the third-party loggers: the backend is imported lazily and
    only rank 0 talks to it."""

    _package = ""
    _hint = ""

    def _import(self):
        import importlib

        try:
            return importlib.import_module(self._package)
        except ImportError as exc:
            raise ImportError(f"``{self._package}`` package not found. {self._hint}") from exc

    @property
    def _active(self) -> bool:
        return get_world_size_and_rank()[1] == 0

    def log(self, name: str, data: Scalar, step: int) -> None:
        self.log_dict({name: data}, step)


class WandBLogger(_RankZeroBackend):
    _package, _hint = "wandb", "Please install wandb using `pip install wandb` to use WandBLogger."

    def __init__(self, project: str = "torchtune", entity: Optional[str] = None, group: Optional[str] = None, log_dir: Optional[str] = None, **kwargs):
        self._wandb = self._import()
        self.log_dir = kwargs.pop("dir", log_dir)
        if self._active and self._wandb.run is None:
            self._wandb.init(project=project, entity=entity, group=group, dir=self.log_dir, **kwargs)
        if self._active and self._wandb.run:
            self._wandb.run._label(repo="torchtune")
            if hasattr(self._wandb, "define_metric"):
                self._wandb.define_metric("global_step")
                self._wandb.define_metric("*", step_metric="global_step", step_sync=True)
        self.config_allow_val_change = kwargs.get("allow_val_change", False)

    def log_config(self, config: DictConfig) -> None:
        if not (self._active and self._wandb.run):
            return
        self._wandb.config.update(OmegaConf.to_container(config, resolve=True), allow_val_change=self.config_allow_val_change)
        path = save_config(config)
        try:
            self._wandb.save(str(path), base_path=str(path.parent))
        except Exception as exc:
            log.warning(f"Error uploading {path} to W&B.\nError: \n{exc}.")

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        if self._active and self._wandb.run:
            self._wandb.log({**payload, "global_step": step})

    def close(self) -> None:
        if self._active and self._wandb.run:
            self._wandb.finish()


class TensorBoardLogger(_RankZeroBackend):
    def __init__(self, log_dir: str, organize_logs: bool = True, **kwargs):
        from torch.utils.tensorboard import SummaryWriter

        self._writer = None
        self.log_dir = os.path.join(log_dir, f"run_{_rank0_time()}") if organize_logs else log_dir
        if self._active:
            self._writer = SummaryWriter(log_dir=self.log_dir)

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        if self._writer:
            for k, v in payload.items():
                self._writer.add_scalar(k, _scalar(v), global_step=step, new_style=True)

    def log_config(self, config: DictConfig) -> None:
        save_config(config)

    def close(self) -> None:
        if self._writer:
            self._writer.close()
            self._writer = None


def _rank0_time() -> float:
    t = time.time()
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        holder = [t]
        torch.distributed.broadcast_object_list(holder, src=0)
        t = holder[0]
    return t


class CometLogger(_RankZeroBackend):
    _package, _hint = "comet_ml", "Please install comet_ml using `pip install comet_ml` to use CometLogger."

    def __init__(self, api_key=None, workspace=None, project=None, experiment_key=None, mode=None, online=None, experiment_name=None, tags=None, log_code=True, **kwargs):
        comet = self._import()
        self.experiment = None
        if self._active:
            self.experiment = comet.start(
                api_key=api_key, workspace=workspace, project=project, experiment_key=experiment_key, mode=mode, online=online,
                experiment_config=comet.ExperimentConfig(log_code=log_code, tags=tags, name=experiment_name, **kwargs),
            )

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        if self.experiment is not None:
            self.experiment.log_metrics(dict(payload), step=step)

    def log_config(self, config: DictConfig) -> None:
        if self.experiment is not None:
            self.experiment.log_parameters(OmegaConf.to_container(config, resolve=True))
            path = save_config(config)
            try:
                self.experiment.log_asset(str(path), file_name="torchtune_config.yaml")
            except Exception as exc:
                log.warning(f"Failed to upload config to Comet assets. Error: {exc}")

    def close(self) -> None:
        if self.experiment is not None:
            self.experiment.end()


class MLFlowLogger(_RankZeroBackend):
    _package, _hint = "mlflow", "Please install mlflow using `pip install mlflow` to use MLFlowLogger."

    def __init__(self, experiment_name: Optional[str] = None, tracking_uri: Optional[str] = None, run_id: Optional[str] = None, run_name: Optional[str] = None):
        self._mlflow = self._import()
        self._run_id = None
        if self._active:
            if tracking_uri:
                self._mlflow.set_tracking_uri(tracking_uri)
            if experiment_name:
                self._mlflow.set_experiment(experiment_name)
            run = self._mlflow.start_run(run_id=run_id, run_name=run_name)
            self._run_id = run.info.run_id

    def log_config(self, config: DictConfig) -> None:
        if self._run_id is None:
            return
        flat = _flatten(OmegaConf.to_container(config, resolve=True))
        self._mlflow.log_params(flat, run_id=self._run_id)
        path = save_config(config)
        if path.is_file():
            self._mlflow.log_artifact(str(path), run_id=self._run_id)

    def log_dict(self, payload: Mapping[str, Scalar], step: int) -> None:
        if self._run_id is not None:
            self._mlflow.log_metrics({k: _scalar(v) for k, v in payload.items()}, step=step, run_id=self._run_id)

    def close(self) -> None:
        if self._run_id is not None:
            self._mlflow.end_run()
            self._run_id = None


def _flatten(d: Dict[str, Any], prefix: str = "") -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for k, v in d.items():
        key = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, dict):
            out.update(_flatten(v, key))
        else:
            out[key] = v
    return out
