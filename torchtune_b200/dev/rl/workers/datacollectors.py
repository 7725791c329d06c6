"""Inference role (parity: torchtune/dev/rl/workers/datacollectors/sync.py:35-411): sample ``group_size`` completions for every
prompt with the newest policy weights this worker has and hand the groups to post-processing."""
from __future__ import annotations

import queue
from typing import Any, Callable, Dict, Iterator, List, Optional

import torch
from torch import nn

from .... import generation
from ....modules.common_utils import delete_kv_caches
from ..datatypes import CompletionOutput, RequestOutput, Trajectory
from .weight_updaters import WeightUpdateReceiver


def _left_pad(tokens: torch.Tensor, pad_id: int) -> torch.Tensor:
    out = torch.full_like(tokens, pad_id)
    for i, n in enumerate((tokens != pad_id).sum(1).tolist()):
        if n:
            out[i, tokens.shape[1] - n :] = tokens[i, :n]
    return out


class SyncLLMCollector:
    def __init__(self, *, model: nn.Module, tokenizer, prompts: Iterator[Dict[str, Any]], rollout_queue, receiver: Optional[WeightUpdateReceiver], device: torch.device,
                 dtype: torch.dtype, group_size: int, max_generated_tokens: int, temperature: float = 1.0, top_k: Optional[int] = None, stop_token_ids: Optional[List[int]] = None,
                 seed: int = 0, worker_id: int = 0, metric_logger=None, steps_before_weight_sync: int = 1):
        self.model, self.tokenizer, self.prompts, self.rollout_queue, self.receiver = model.eval(), tokenizer, prompts, rollout_queue, receiver
        self.device, self.dtype, self.group_size, self.max_generated_tokens = device, dtype, group_size, max_generated_tokens
        self.temperature, self.top_k = temperature, top_k
        self.pad_id = getattr(tokenizer, "pad_id", 0)
        self.stop_token_ids = list(stop_token_ids if stop_token_ids is not None else getattr(tokenizer, "stop_tokens", []) or [])
        self.rng = torch.Generator(device).manual_seed(seed)
        self.worker_id, self.metric_logger, self.steps_before_weight_sync = worker_id, metric_logger, max(1, steps_before_weight_sync)
        self.batches_done = 0

    @torch.no_grad()
    def generate(self, prompt_tokens: torch.Tensor, answers: List[str], request_ids: Optional[List[str]] = None) -> List[RequestOutput]:
        """``prompt_tokens`` ``[b, P]`` right-padded → one :class:`RequestOutput` with ``group_size`` completions per prompt."""
        b, ctx = prompt_tokens.shape
        g = self.group_size
        batch = _left_pad(prompt_tokens.to(self.device), self.pad_id)[:, None, :].expand(b, g, ctx).reshape(b * g, ctx)
        self.model.setup_caches(batch_size=b * g, dtype=self.dtype, decoder_max_seq_len=ctx + self.max_generated_tokens)
        try:
            tokens, logits = generation.generate(model=self.model, prompt=batch, max_generated_tokens=self.max_generated_tokens, temperature=self.temperature, top_k=self.top_k,
                                                 pad_id=self.pad_id, rng=self.rng, stop_tokens=self.stop_token_ids or None)
        finally:
            delete_kv_caches(self.model)
        responses = tokens[:, ctx:]
        logp = torch.log_softmax(logits.float() / max(self.temperature, 1e-6), dim=-1).gather(-1, responses.unsqueeze(-1)).squeeze(-1)
        version = self.receiver.version if self.receiver is not None else 0
        out: List[RequestOutput] = []
        stop = set(self.stop_token_ids)
        for i in range(b):
            req = RequestOutput(request_id=(request_ids[i] if request_ids else f"w{self.worker_id}-b{self.batches_done}-p{i}"), prompt_token_ids=batch[i * g].tolist(), answer=answers[i],
                                policy_version=version)
            for j in range(g):
                row = responses[i * g + j].tolist()
                n, reason = len(row), "length"
                for t, tok in enumerate(row):
                    if tok in stop:
                        n, reason = t + 1, "stop"
                        break
                    if tok == self.pad_id and self.pad_id not in stop:
                        n, reason = t, "stop"
                        break
                req.outputs.append(CompletionOutput(index=j, token_ids=row[:n], logprobs=logp[i * g + j, :n].tolist(), finish_reason=reason))
            out.append(req)
        return out

    def to_trajectory(self, req: RequestOutput) -> Trajectory:
        responses, logprobs, pad = req.padded(self.max_generated_tokens, self.pad_id)
        g = responses.shape[0]
        prompt = torch.tensor(req.prompt_token_ids, dtype=torch.long).unsqueeze(0).expand(g, -1)
        qr = torch.cat([prompt, responses], dim=1)
        real = torch.cat([prompt != self.pad_id, ~pad], dim=1)
        return Trajectory(query_responses=qr, responses=responses, logprobs=logprobs, ref_logprobs=None, query_response_padding_masks=real, seq_lens=(~pad).sum(1), answers=[req.answer] * g,
                          policy_version=req.policy_version, sequence_ids=[f"{req.request_id}-{j}" for j in range(g)])

    def run(self, stop_event, max_batches: Optional[int] = None) -> None:
        """Until told to stop (or the prompts run out): sync weights every ``steps_before_weight_sync`` batches, generate, enqueue."""
        for batch in self.prompts:
            if stop_event.is_set() or (max_batches is not None and self.batches_done >= max_batches):
                return
            if self.receiver is not None and self.batches_done % self.steps_before_weight_sync == 0:
                self.receiver.maybe_update()
            for req in self.generate(batch["tokens"], list(batch["answers"])):
                traj = self.to_trajectory(req)
                while not stop_event.is_set():
                    try:
                        self.rollout_queue.put(traj, timeout=0.2)
                        break
                    except queue.Full:
                        continue
            self.batches_done += 1
            if self.metric_logger is not None:
                self.metric_logger.log_dict({f"inference/worker_{self.worker_id}/batches": self.batches_done,
                                             f"inference/worker_{self.worker_id}/policy_version": self.receiver.version if self.receiver else 0}, step=self.batches_done)


class GeneratorWeightWorker:
    """Receiving end of :class:`~torchtune_b200.dev.rl.workers.parameter_servers.BroadcastParameterServer`
    (parity: torchtune/dev/rl/workers/datacollectors/sync.py:368-411, the worker the reference plugs into its inference engine).

    Wraps the model this package's own generator runs.  ``init_weight_update_group`` joins the update group at rank
    ``local_rank + rank_offset`` (the server is rank 0, so the offset is at least 1); ``update_weight`` receives one tensor and loads
    it; ``update_policy_version`` receives the version.  ``receive`` does a whole push: the version, then every tensor of the model's
    state dict in sorted-name order."""

    def __init__(self, model: nn.Module, device: Optional[torch.device] = None, local_rank: int = 0):
        self.model, self.local_rank = model, int(local_rank)
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.version = 0
        self._group = None

    def init_weight_update_group(self, master_address: str, master_port: int, rank_offset: int, world_size: int, timeout_s: float = 600.0) -> None:
        from ..utils import stateless_init_process_group

        if rank_offset < 1:
            raise ValueError("rank 0 of the update group belongs to the parameter server")
        self._group = stateless_init_process_group(master_address, master_port, self.local_rank + rank_offset, world_size,
                                                   self.device if self.device.type == "cuda" else None, timeout_s)

    def update_weight(self, name: str, dtype: torch.dtype, shape) -> None:
        buf = torch.empty(tuple(shape), dtype=dtype, device=self._group.device)
        self._group.broadcast(buf, src=0)
        target = self.model.state_dict(keep_vars=True)[name]
        with torch.no_grad():
            target.copy_(buf)

    def update_policy_version(self) -> int:
        v = torch.zeros(1, dtype=torch.int64, device=self._group.device)
        self._group.broadcast(v, src=0)
        self.version = int(v.item())
        return self.version

    def receive(self) -> int:
        """One whole push from the server; returns the new policy version."""
        if self._group is None:
            raise RuntimeError("init_weight_update_group() has not been called")
        self.update_policy_version()
        state = self.model.state_dict(keep_vars=True)
        for name in sorted(state):
            self.update_weight(name, state[name].dtype, state[name].shape)
        return self.version

    def close(self) -> None:
        if self._group is not None:
            self._group.close()
            self._group = None


# the reference's name for this role
VLLMWorkerWrapper = GeneratorWeightWorker
