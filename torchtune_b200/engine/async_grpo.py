"""Controller of the asynchronous GRPO recipe (reference: recipes/dev/async_grpo_full_finetune_distributed.py:118-315, a Ray
program that places vLLM inference workers, a reference-model worker, FSDP trainers, a parameter server and a metric logger).

The same roles (:mod:`torchtune_b200.dev.rl.workers`) are wired with queues.  ``orchestration.backend: thread`` runs every role as
a thread of this process (roles on different GPUs still overlap, because kernels are launched asynchronously and the host work of
one role releases the interpreter lock while another waits on its device).  ``orchestration.backend: process`` moves the inference
workers — the host-bound roles: one Python decoding loop each — into child processes: trajectories come back through a
``multiprocessing`` queue, the parameter server keeps the weights in shared memory under a process lock with a shared version
counter (the children pull newer weights between batches), metrics and failures travel over queues, one shared event stops
everybody.  Post-processing, trainer and logger stay threads of the controller.  Inference workers take disjoint shards of the
prompt dataset.  Data flow:

    prompts → [SyncLLMCollector × num_inference_workers] → rollout queue → [PostProcessingWorker × num_postprocessing_workers]
            → replay buffer → TrainingWorker → ParameterServer → (weights, version) → collectors

The trainer runs ``orchestration.num_steps`` steps and then raises the stop flag; ``train/policy_staleness`` (trainer version
minus the version that sampled a batch) is logged with every step.  Devices: ``inference.devices`` / ``postprocessing.devices`` /
``training.device`` name one device per worker; by default workers are spread over the visible GPUs (CPU without any).
"""
from __future__ import annotations

import itertools
import queue
import threading
from functools import partial
from typing import Any, Dict, List, Optional

import torch

from .. import config, modules, training, utils
from ..config import DictConfig
from ..dev.grpo import padded_collate_rl
from ..dev.rl.workers import MetricLoggerWorker, ParameterServer, PostProcessingWorker, ReplayBuffer, SyncLLMCollector, TrainingWorker, WeightUpdateReceiver
from .dataloading import StatefulDataLoader, StatefulDistributedSampler

log = utils.get_logger("DEBUG")


def _device_list(spec: Any, n: int, offset: int) -> List[torch.device]:
    if spec:
        names = [spec] * n if isinstance(spec, str) else list(spec)
        if len(names) != n:
            raise ValueError(f"expected {n} devices, got {names}")
        return [torch.device(d) for d in names]
    if not torch.cuda.is_available():
        return [torch.device("cpu")] * n
    count = torch.cuda.device_count()
    return [torch.device("cuda", (offset + i) % count) for i in range(n)]


class _QueueMetricLogger:
    """Stands in for the metric-logger worker inside a child process: forwards every record over a queue."""

    def __init__(self, q):
        self.q = q

    def log_dict(self, payload: Dict[str, Any], step: int) -> None:
        try:
            self.q.put_nowait(({k: float(v) for k, v in payload.items()}, int(step)))
        except queue.Full:
            pass


def _inference_process(cfg_container: Dict[str, Any], index: int, n_workers: int, seed: int, device_name: str, dtype_name: str, server: ParameterServer, rollout_q, metrics_q, error_q,
                       stop_event) -> None:
    """Body of one inference worker run as a child process (``orchestration.backend: process``)."""
    try:
        cfg = config.OmegaConf.create(cfg_container)
        inf = cfg.inference
        device, dtype = torch.device(device_name), getattr(torch, dtype_name)
        torch.set_num_threads(max(1, torch.get_num_threads() // max(1, n_workers)))
        tokenizer = config.instantiate(cfg.tokenizer)
        pad_id = getattr(tokenizer, "pad_id", 0)
        ds = config.instantiate(cfg.dataset, tokenizer)
        sampler = StatefulDistributedSampler(ds, num_replicas=n_workers, rank=index, shuffle=cfg.get("shuffle", False), seed=seed)
        loader = StatefulDataLoader(ds, batch_size=int(inf.get("batch_size", 1)), sampler=sampler, collate_fn=partial(padded_collate_rl, padding_idx=pad_id), drop_last=True)
        with training.set_default_dtype(dtype), device:
            policy = config.instantiate(cfg.model)
        _, weights = server.fetch(-1)  # the weights the server was created with (version 0) or whatever is newest by now
        policy.load_state_dict(weights)
        collector = SyncLLMCollector(model=policy, tokenizer=tokenizer, prompts=itertools.chain.from_iterable(itertools.repeat(loader)), rollout_queue=rollout_q,
                                     receiver=WeightUpdateReceiver(server, policy), device=device, dtype=dtype, group_size=int(inf.group_size),
                                     max_generated_tokens=int(inf.max_generated_tokens), temperature=float(inf.get("temperature", 1.0)), top_k=inf.get("top_k"),
                                     seed=seed + 1000 * (index + 1), worker_id=index, metric_logger=_QueueMetricLogger(metrics_q),
                                     steps_before_weight_sync=int(inf.get("steps_before_weight_sync", 1)))
        collector.run(stop_event)
    except BaseException as exc:  # noqa: BLE001  reported to the controller, which stops the job
        import traceback

        error_q.put(f"inference worker {index}: {exc!r}\n{traceback.format_exc()}")
        stop_event.set()
    finally:
        rollout_q.cancel_join_thread()  # trajectories nobody will read any more must not keep the process alive
        metrics_q.cancel_join_thread()


class AsyncGRPORecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self.cfg = cfg
        orch = cfg.orchestration
        self.num_inference_workers = int(orch.num_inference_workers)
        self.num_postprocessing_workers = int(orch.get("num_postprocessing_workers", 1))
        self.num_training_workers = int(orch.get("num_training_workers", 1))
        if self.num_training_workers != 1:
            raise NotImplementedError("the controller drives one training worker; for data-parallel training of the policy launch the synchronous "
                                      "recipe dev/grpo_full_finetune_distributed under `tune run --nproc_per_node N`")
        self.backend = str(orch.get("backend", "thread"))
        if self.backend not in ("thread", "process"):
            raise ValueError("orchestration.backend must be 'thread' or 'process'")
        self.seed = training.set_seed(seed=cfg.training.get("seed"))
        if self.backend == "process":
            import torch.multiprocessing as mp

            self._mp = mp.get_context("spawn")
            self.stop_event = self._mp.Event()
        else:
            self._mp = None
            self.stop_event = threading.Event()
        self.threads: List[threading.Thread] = []
        self.processes: list = []
        self.errors: List[BaseException] = []

    # ------------------------------------------------------------------ setup
    def _build_model(self, device: torch.device, dtype: torch.dtype, state_dict: Dict[str, torch.Tensor]) -> torch.nn.Module:
        with training.set_default_dtype(dtype), device:
            model = config.instantiate(self.cfg.model)
        model.load_state_dict(state_dict)
        return model

    def setup(self, cfg: Optional[DictConfig] = None) -> None:
        cfg = cfg or self.cfg
        inf, post, trn = cfg.inference, cfg.postprocessing, cfg.training
        dtype = training.get_dtype(cfg.get("dtype"), device=utils.get_device(cfg.get("device")))
        self.metric_logger = MetricLoggerWorker(config.instantiate(cfg.metric_logger))
        self.metric_logger.logger.log_config(cfg)
        self.tokenizer = config.instantiate(cfg.tokenizer)
        pad_id = getattr(self.tokenizer, "pad_id", 0)
        self.checkpointer = config.instantiate(trn.checkpointer, should_load_recipe_state=False)
        policy_sd = self.checkpointer.load_checkpoint()[training.MODEL_KEY]
        ref_sd = config.instantiate(post.ref_checkpointer, should_load_recipe_state=False).load_checkpoint()[training.MODEL_KEY]

        n_inf, n_post = self.num_inference_workers, self.num_postprocessing_workers
        inf_devices = _device_list(inf.get("devices"), n_inf, 0)
        post_devices = _device_list(post.get("devices"), n_post, n_inf)
        train_device = _device_list(trn.get("device"), 1, n_inf + n_post)[0]

        group_size, batch_size = int(inf.group_size), int(inf.get("batch_size", 1))
        self.replay_buffer = ReplayBuffer(int(cfg.orchestration.get("replay_buffer_size", batch_size)))
        if self.backend == "process":
            self.rollout_queue = self._mp.Queue(maxsize=int(inf.get("queue_maxsize", n_inf)))
            self.metrics_queue, self.error_queue = self._mp.Queue(maxsize=1024), self._mp.Queue()
            self.param_server = ParameterServer(policy_sd, shared=True, lock=self._mp.Lock(), version=self._mp.Value("i", 0))
        else:
            self.rollout_queue = queue.Queue(maxsize=int(inf.get("queue_maxsize", n_inf)))
            self.param_server = ParameterServer(policy_sd)

        # training role
        model = self._build_model(train_device, dtype, policy_sd)
        if trn.get("enable_activation_checkpointing", False):
            training.set_activation_checkpointing(model, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
        training.disable_dropout(model)
        optimizer = config.instantiate(trn.optimizer, list(model.parameters()))
        loss_fn = config.instantiate(trn.loss)
        offload = training.get_act_offloading_ctx_manager(model, True) if (trn.get("enable_activation_offloading", False) and train_device.type == "cuda") else None
        groups_per_step = max(1, int(trn.get("batch_size", group_size)) // group_size)
        self.trainer = TrainingWorker(model=model, optimizer=optimizer, loss_fn=loss_fn, replay_buffer=self.replay_buffer, param_server=self.param_server, device=train_device,
                                      batch_groups=groups_per_step, num_steps=int(cfg.orchestration.num_steps), ppo_epochs=int(trn.get("ppo_epochs", 1)),
                                      clip_grad_norm=trn.get("clip_grad_norm"), steps_before_weight_sync=int(trn.get("steps_before_weight_sync", 1)), metric_logger=self.metric_logger,
                                      pad_id=pad_id, save_fn=self._save, save_every_n_steps=trn.get("save_every_n_steps"), activations_ctx=offload)

        # post-processing roles
        rewards = [config.instantiate(r) for r in cfg.reward_functions]
        self.postprocessors = [PostProcessingWorker(ref_model=self._build_model(d, dtype, ref_sd), tokenizer=self.tokenizer, reward_functions=rewards, rollout_queue=self.rollout_queue,
                                                    replay_buffer=self.replay_buffer, device=d, temperature=float(inf.get("temperature", 1.0)), metric_logger=self.metric_logger, worker_id=i)
                               for i, d in enumerate(post_devices)]

        # inference roles: every worker reads its own shard of the prompts, for as many passes as the run lasts
        self.collectors = []
        if self.backend == "process":
            container = config.OmegaConf.to_container(cfg, resolve=True)
            dtype_name = str(dtype).replace("torch.", "")
            for i, d in enumerate(inf_devices):
                self.processes.append(self._mp.Process(target=_inference_process, name=f"inference-{i}", daemon=True,
                                                       args=(container, i, n_inf, self.seed, str(d), dtype_name, self.param_server, self.rollout_queue, self.metrics_queue,
                                                             self.error_queue, self.stop_event)))
            return
        ds = config.instantiate(cfg.dataset, self.tokenizer)
        for i, d in enumerate(inf_devices):
            sampler = StatefulDistributedSampler(ds, num_replicas=n_inf, rank=i, shuffle=cfg.get("shuffle", False), seed=self.seed)
            loader = StatefulDataLoader(ds, batch_size=batch_size, sampler=sampler, collate_fn=partial(padded_collate_rl, padding_idx=pad_id), drop_last=True)
            policy = self._build_model(d, dtype, policy_sd)
            self.collectors.append(SyncLLMCollector(model=policy, tokenizer=self.tokenizer, prompts=itertools.chain.from_iterable(itertools.repeat(loader)), rollout_queue=self.rollout_queue,
                                                    receiver=WeightUpdateReceiver(self.param_server, policy), device=d, dtype=dtype, group_size=group_size,
                                                    max_generated_tokens=int(inf.max_generated_tokens), temperature=float(inf.get("temperature", 1.0)), top_k=inf.get("top_k"),
                                                    seed=self.seed + 1000 * (i + 1), worker_id=i, metric_logger=self.metric_logger,
                                                    steps_before_weight_sync=int(inf.get("steps_before_weight_sync", 1))))

    # ------------------------------------------------------------------ run
    def _spawn(self, name: str, fn, *args) -> None:
        def guarded():
            try:
                fn(*args)
            except BaseException as exc:  # noqa: BLE001  a role that dies stops the whole job instead of leaving the others waiting
                self.errors.append(exc)
                self.stop_event.set()

        t = threading.Thread(target=guarded, name=name, daemon=True)
        t.start()
        self.threads.append(t)

    def _pump_children(self) -> None:
        """Controller-side thread of the process backend: records of the children go to the metric logger, the first reported failure
        stops the job, and so does a child that exits on its own."""
        while not self.stop_event.is_set():
            try:
                payload, step = self.metrics_queue.get(timeout=0.2)
                self.metric_logger.log_dict(payload, step=step)
            except queue.Empty:
                pass
            try:
                self.errors.append(RuntimeError(self.error_queue.get_nowait()))
                self.stop_event.set()
            except queue.Empty:
                pass
            for p in self.processes:
                if p.exitcode not in (None, 0):
                    self.errors.append(RuntimeError(f"{p.name} exited with code {p.exitcode}"))
                    self.stop_event.set()

    def train(self) -> None:
        self._spawn("metric-logger", self.metric_logger.run, self.stop_event)
        for p in self.processes:
            p.start()
        if self.processes:
            self._spawn("children", self._pump_children)
        for i, c in enumerate(self.collectors):
            self._spawn(f"inference-{i}", c.run, self.stop_event)
        for i, p in enumerate(self.postprocessors):
            self._spawn(f"postprocessing-{i}", p.run, self.stop_event)
        self._spawn("training", self.trainer.run, self.stop_event)
        for t in self.threads:
            while t.is_alive():
                t.join(timeout=0.5)
        for p in self.processes:  # the stop flag is set by now: a child leaves its loop after the batch it is working on
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
        if self.errors:
            raise RuntimeError(f"a worker failed: {self.errors[0]!r}") from self.errors[0]
        self._save(self.trainer, self.trainer.step, final=True)

    def _save(self, trainer: TrainingWorker, step: int, final: bool = False) -> None:
        sd = {k: v.detach().cpu() for k, v in trainer.model.state_dict().items()}
        self.checkpointer.save_checkpoint({training.MODEL_KEY: sd}, epoch=0, intermediate_checkpoint=False, step=step if not final else None)

    def cleanup(self) -> None:
        self.stop_event.set()
        self.metric_logger.close()
