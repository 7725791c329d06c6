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

from typing import Any, Dict, Optional

import torch
from torch import nn

from ..ops.mask import AttentionMask
from ..utils import batch_to_device


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

    def _step_done(self) -> None:
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
