"""One optimisation step as a callable: host batch in, loss out.

``TrainStep`` is the smallest public unit a user drives directly (the recipes' loops are
built from the same pieces): it uploads a batch from (pinned) host memory, runs forward and
backward through the sm_100a kernels, normalises by the global number of unmasked label
tokens, steps the optimizer and returns the mean token loss as a device scalar — the
caller decides when to synchronise (``.item()``).

Token accounting follows the reference recipes: the summed loss is back-propagated and the
gradients are divided by the all-reduced token count inside the optimizer update
(recipes/full_finetune_distributed.py:1007-1039).
"""
from __future__ import annotations

import gc
import os
import weakref
from typing import Any, Dict, Optional

import torch
from torch import nn

from ..ops.mask import AttentionMask
from ..utils import batch_to_device


class HostGarbageControl:
    """Keeps the cyclic garbage collector from pausing the host in the middle of a step.  Python's generational collector starts
    whenever allocation counts cross a threshold; a full collection with a model's worth of live objects can hold the launching
    thread for long enough that the device queue runs dry.  Training state is not cyclic garbage, so automatic collection is
    switched off and a generation-1 collection runs every ``period`` steps at a step boundary instead.  ``TTB_HOST_GC=auto``
    leaves Python's own schedule in place."""

    def __init__(self, active: bool = True, period: int = 50):
        self.period = period
        self.enabled = active and os.environ.get("TTB_HOST_GC", "manual") != "auto" and gc.isenabled()
        self._count = 0
        if self.enabled:
            gc.collect()
            gc.freeze()  # what is alive now (model, optimizer, data) is never scanned again
            gc.disable()
            weakref.finalize(self, HostGarbageControl._restore)

    @staticmethod
    def _restore() -> None:
        gc.enable()
        gc.unfreeze()

    def step(self) -> None:
        if not self.enabled:
            return
        self._count += 1
        if self._count % self.period == 0:
            gc.collect(1)

    def close(self) -> None:
        if self.enabled:
            self._restore()
            self.enabled = False


class TrainStep:
    def __init__(self, model: nn.Module, loss_fn, optimizer, device: torch.device, parallel=None, clip_grad_norm: Optional[float] = None, activations_ctx=None):
        self.model, self.loss_fn, self.optimizer = model, loss_fn, optimizer
        # context entered around the forward pass (``training.get_act_offloading_ctx_manager``: pinned-host activation offload)
        self.activations_ctx = activations_ctx
        self.device = device
        self.parallel = parallel
        self.clip_grad_norm = clip_grad_norm
        self._params = [p for p in model.parameters() if p.requires_grad]
        self.max_steps_in_flight = 2
        self._in_flight: list = []
        self.trace_events = None  # set to a list to collect one CUDA event per phase boundary of every step
        self.host_gc = HostGarbageControl(active=device.type == "cuda")  # CPU runs (tests) keep Python's own schedule

    def _step_done(self) -> None:
        self.host_gc.step()
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._in_flight.append(ev)

    def _mark(self) -> None:
        """Phase boundaries as CUDA events when ``trace_events`` is a list (forward+loss, backward, token all-reduce, optimizer)."""
        if self.trace_events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace_events.append(ev)

    def upload(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        out = dict(batch)
        batch_to_device(out, self.device)
        return out

    def compute(self, batch: Dict[str, Any]) -> torch.Tensor:
        """Forward, backward and update on a batch that already lives on the device."""
        batch = dict(batch)
        labels = batch.pop("labels")
        # Bound how far the host runs ahead of the device: wait for the step before the previous one.  One full step of work
        # stays queued, so the device never idles, but launch queues do not grow without limit (deep queues across the
        # training, weight-gradient and communication streams produced sporadic stalls of several hundred milliseconds).
        if self.device.type == "cuda":
            if len(self._in_flight) >= self.max_steps_in_flight:
                self._in_flight.pop(0).synchronize()
        self._mark()
        if hasattr(self.model, "shard_rows"):  # tensor + sequence parallel model: the loss runs on this rank's token rows
            labels = self.model.shard_rows(labels)
        if self.activations_ctx is not None:
            with self.activations_ctx:
                hidden = self.model(**batch)
                loss_sum, n_valid = self.loss_fn.compute_sum(hidden, labels)
        else:
            hidden = self.model(**batch)
            loss_sum, n_valid = self.loss_fn.compute_sum(hidden, labels)
        self._mark()
        n_tokens = n_valid.to(torch.float32)
        if self.parallel is not None:
            total = loss_sum.detach().clone()
            overlap = getattr(self.parallel, "wants_backward_overlap", lambda _o: False)(self.optimizer)
            if overlap:
                # the global token count is final before backward, so the optimizer can consume each layer's gradients while
                # backward is still running on the earlier layers
                self.parallel.all_reduce_sum_(n_tokens, total)
                self.parallel.arm_backward_overlap(self.optimizer, 1.0 / n_tokens, self.clip_grad_norm)
            loss_sum.backward()
            self._mark()
            if not overlap:
                self.parallel.all_reduce_sum_(n_tokens, total)
            self._mark()
            self.parallel.optimizer_step(self.model, self.optimizer, 1.0 / n_tokens, self.clip_grad_norm)
            self._mark()
            self._step_done()
            return total / n_tokens
        loss_sum.backward()
        self.optimizer.step(grad_scale=1.0 / n_tokens, max_grad_norm=self.clip_grad_norm)
        self.optimizer.zero_grad(set_to_none=True)
        self._step_done()
        return loss_sum.detach() / n_tokens

    def __call__(self, host_batch: Dict[str, Any]) -> torch.Tensor:
        return self.compute(self.upload(host_batch))
