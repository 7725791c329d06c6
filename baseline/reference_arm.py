"""Reference arm of ``bench.py``: the unmodified reference implementation (installed under
``baseline/_ref`` with ``pip --no-deps --target``) on the benchmark configuration.

The code below only *drives* the reference through its public Python API and follows the
stock path of its full-finetune recipes step by step
(recipes/full_finetune_single_device.py / recipes/full_finetune_distributed.py):

  model      torchtune.models.llama3_1.llama3_1(...)            (same hyper-parameters as ours)
  AC         torchtune.training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
  FSDP (N>1) torchtune.training.shard_model(..., get_shard_conditions(tok_embeddings, output))
  mask       torchtune.modules.attention_utils.packed_block_causal_mask(seq_lens)  → flex attention
  loss       torchtune.modules.loss.LinearCrossEntropyLoss + set_model_output
  optimizer  torch.optim.AdamW(lr=2e-5, fused=True)
  step       loss·n_tokens backward → all-reduce n_tokens → training.scale_grads_(world/n) → step

``run_peft`` does the same for the adapter configurations (``bench.py --variant lora | dpo``), following
recipes/lora_finetune_single_device.py / recipes/lora_finetune_distributed.py and recipes/lora_dpo_distributed.py:

  model      torchtune.models.llama3_1.lora_llama3_1_8b(q,k,v,output_proj + MLP, r=64, alpha=128)
  trainable  set_trainable_params(model, get_adapter_params(model))
  FSDP (N>1) training.shard_model(...) on the meta-device model, adapters ``to_empty`` + ``initialize_parameters``
  DPO        logits = model(tokens) → rlhf.get_batch_log_probs; reference pass under no_grad + disable_adapter;
             torchtune.rlhf.loss.DPOLoss(beta=0.1); loss.mean().backward(); optimizer.step()

The QLoRA reference needs ``torchao.quantization.to_nf4`` (torchtune/modules/peft/lora.py:15,86); torchao is not installed, so
that arm reports ``unavailable``.

None of this repository's models, kernels or engine are imported.  ``torchao`` and
``omegaconf`` are absent from this image and the reference refuses to import without them, so
inert import-time placeholders are registered first (``baseline/shims/missing_deps.py``); the
bf16 path exercised here never calls into either package.
"""
from __future__ import annotations

import os
import sys
from functools import partial
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _import_reference():
    ref_dir = HERE / "_ref"
    if not (ref_dir / "torchtune").is_dir():
        raise ImportError(f"{ref_dir} does not contain the reference install")
    sys.path.insert(0, str(HERE / "shims"))
    sys.path.insert(0, str(ref_dir))
    import missing_deps

    missing_deps.install()
    import torchtune  # noqa: F401

    return torchtune


def run(args, model_cfg, seq_len, doc_len, batch_per_gpu, lr, ClockSampler, timed_loop, dist_env) -> dict:
    try:
        _import_reference()
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference cannot be imported: {type(exc).__name__}: {exc}"[:300]}

    import torch
    import torch.distributed as dist
    from torchtune import modules, training
    from torchtune.models.llama3_1 import llama3_1
    from torchtune.modules.attention_utils import packed_block_causal_mask
    from torchtune.modules.loss import LinearCrossEntropyLoss

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1234)

    init_device = torch.device("meta") if world > 1 else device
    with training.set_default_dtype(torch.bfloat16), init_device:
        model = llama3_1(**model_cfg)
    compiled = bool(getattr(args, "ref_compile", False))
    if compiled:  # informational arm: the recipe's ``compile: True`` (per-layer torch.compile of the model, compiled loss)
        training.compile_model(model, verbose=False)
    training.set_activation_checkpointing(model, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
    if world > 1:
        conditions = [partial(training.get_shard_conditions, names_to_match=["tok_embeddings", "output"])]
        training.shard_model(model=model, shard_conditions=conditions, cpu_offload=False, reshard_after_forward=True)
        model.to_empty(device=device)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                torch.nn.init.normal_(p, std=0.02)
            else:
                p.fill_(1.0)
        for m in model.modules():
            if hasattr(m, "rope_init"):
                with device:
                    m.rope_init()
    loss_fn = LinearCrossEntropyLoss()
    if compiled:
        loss_fn = training.compile_loss(loss_fn, verbose=False)
    loss_fn.set_model_output(model)
    optimizer = torch.optim.AdamW(model.parameters(), lr=lr, fused=True)

    n_docs = seq_len // doc_len

    def host_batch(seed):
        g = torch.Generator().manual_seed(seed)
        tokens = torch.randint(0, model_cfg["vocab_size"], (batch_per_gpu, seq_len), generator=g, dtype=torch.long)
        labels = torch.roll(tokens, -1, dims=1)
        labels[:, doc_len - 1 :: doc_len] = -100
        pos = torch.arange(doc_len).repeat(n_docs).unsqueeze(0).expand(batch_per_gpu, seq_len).contiguous()
        seq_lens = torch.full((batch_per_gpu, n_docs), doc_len, dtype=torch.long)
        return {"tokens": tokens.pin_memory(), "labels": labels.pin_memory(), "input_pos": pos.pin_memory(), "seq_lens": seq_lens.pin_memory()}

    def upload(h):
        d = {k: v.to(device, non_blocking=True) for k, v in h.items()}
        d["mask"] = packed_block_causal_mask([row for row in d.pop("seq_lens")])
        return d

    def step(batch):
        batch = dict(batch)
        labels = batch.pop("labels")
        n_tokens = (labels != loss_fn.ignore_index).sum()
        out = model(**batch)
        loss = loss_fn(out, labels) * n_tokens
        loss.backward()
        if world > 1:
            dist.all_reduce(n_tokens)
            dist.all_reduce(loss)
        training.scale_grads_(model.parameters(), world / n_tokens)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss.detach() / n_tokens

    hosts = [host_batch(1000 * rank + i) for i in range(4)]
    devs = [upload(h) for h in hosts]
    for i in range(args.warmup):
        last = step(devs[i % 4])
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    losses = []
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step(devs[i % 4])), args.steps)
    t_e2e = timed_loop(torch, dist, world, lambda i: losses.append(float(step(upload(hosts[i % 4])).item())), args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    tokens_per_step = batch_per_gpu * seq_len * world
    h2d = sum(t.numel() * t.element_size() for t in hosts[0].values())
    value = tokens_per_step * args.steps / t_kernel
    out = {
        "metric": "tokens_per_second",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 * t_kernel / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform tokens, random-init weights",
        "impl": "reference",
        "config": {
            "model": "llama3_1_8b",
            "global_batch": batch_per_gpu * world,
            "seq_len": seq_len,
            "doc_len": doc_len,
            "parallelism": f"fsdp{world}" if world > 1 else "single",
            "activation_checkpointing": True,
            "optimizer": "torch.optim.AdamW fused lr 2e-5",
            "l2": "inputs larger than L2 (16 GB of weights streamed every step)",
            **({"compile": "torch.compile per layer + compiled loss (informational arm, not the stock eager path)"} if compiled else {}),
        },
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": 0,
        "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2),
        "final_loss": float(losses[-1]) if losses else None,
    }
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_peft(args, model_cfg, seq_len, batch_per_gpu, dpo_len, dpo_prompt, dpo_beta, lr, ClockSampler, timed_loop, dist_env) -> dict:
    variant = args.variant
    if variant == "qlora":
        return {"impl": "reference", "unavailable": "the reference's NF4 base weights come from torchao.quantization.to_nf4 (torchtune/modules/peft/lora.py:15,86) and torchao is not installed in this image"}
    try:
        _import_reference()
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference cannot be imported: {type(exc).__name__}: {exc}"[:300]}

    import torch
    import torch.distributed as dist
    from torchtune import modules, rlhf, training
    from torchtune.models.llama3_1 import lora_llama3_1_8b
    from torchtune.modules.loss import LinearCrossEntropyLoss
    from torchtune.modules.peft import AdapterModule, disable_adapter, get_adapter_params, set_trainable_params

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1234)

    init_device = torch.device("meta") if world > 1 else device
    with training.set_default_dtype(torch.bfloat16), init_device:
        model = lora_llama3_1_8b(lora_attn_modules=["q_proj", "k_proj", "v_proj", "output_proj"], apply_lora_to_mlp=True, lora_rank=64, lora_alpha=128)
    set_trainable_params(model, get_adapter_params(model))
    training.set_activation_checkpointing(model, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
    if world > 1:
        conditions = [partial(training.get_shard_conditions, names_to_match=["tok_embeddings", "output"])]
        training.shard_model(model=model, shard_conditions=conditions, cpu_offload=False, reshard_after_forward=True)
        model.to_empty(device=device)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "lora_" in name:
                continue
            if p.dim() > 1:
                torch.nn.init.normal_(p, std=0.02)
            else:
                p.fill_(1.0)
    with training.set_default_dtype(torch.bfloat16), device:
        for m in model.modules():
            if isinstance(m, AdapterModule):
                m.initialize_parameters()
            if hasattr(m, "rope_init"):
                m.rope_init()
    optimizer = torch.optim.AdamW(model.parameters(), lr=lr, fused=True)

    vocab = model_cfg["vocab_size"]
    if variant == "dpo":
        # torchtune/rlhf/loss/dpo.py:14-27 uses TypeVar, dataclass, Optional and Tuple without importing them, so the module does not
        # import as shipped.  The names are made visible through ``builtins`` for the duration of the import; the file stays untouched.
        import builtins
        import dataclasses
        import typing

        injected = {"TypeVar": typing.TypeVar, "dataclass": dataclasses.dataclass, "Optional": typing.Optional, "Tuple": typing.Tuple}
        missing = {k: v for k, v in injected.items() if not hasattr(builtins, k)}
        for k, v in missing.items():
            setattr(builtins, k, v)
        try:
            from torchtune.rlhf.loss import DPOLoss
        finally:
            for k in missing:
                delattr(builtins, k)
        loss_fn = DPOLoss(beta=dpo_beta)

        def host_batch(seed):
            g = torch.Generator().manual_seed(seed)
            prompt = torch.randint(0, vocab, (batch_per_gpu, dpo_prompt), generator=g, dtype=torch.long)
            tails = torch.randint(0, vocab, (2 * batch_per_gpu, dpo_len - dpo_prompt), generator=g, dtype=torch.long)
            tokens = torch.cat([torch.cat([prompt, prompt]), tails], dim=1)
            labels = tokens.clone()
            labels[:, :dpo_prompt] = -100
            return {"tokens": tokens.pin_memory(), "labels": labels.pin_memory()}

        def concatenated_forward(tokens, labels):
            n = tokens.shape[0] // 2
            logits = model(tokens)
            logps = rlhf.get_batch_log_probs(logits, labels)
            return rlhf.ChosenRejectedOutputs(logps[:n], logps[n:], logits[:n], logits[n:])

        def step(batch):
            policy = concatenated_forward(batch["tokens"], batch["labels"])
            policy.chosen_logits = policy.rejected_logits = None
            with torch.no_grad(), disable_adapter(model):
                reference = concatenated_forward(batch["tokens"], batch["labels"])
                reference.chosen_logits = reference.rejected_logits = None
            loss, chosen_rewards, rejected_rewards = loss_fn(policy, reference)
            loss = loss.mean()
            loss.backward()
            if world > 1:
                running = loss.detach().clone()
                dist.all_reduce(running)
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
            return loss.detach()
    else:
        loss_fn = LinearCrossEntropyLoss()
        loss_fn.set_model_output(model)

        def host_batch(seed):
            g = torch.Generator().manual_seed(seed)
            tokens = torch.randint(0, vocab, (batch_per_gpu, seq_len), generator=g, dtype=torch.long)
            labels = torch.roll(tokens, -1, dims=1)
            labels[:, -1] = -100
            return {"tokens": tokens.pin_memory(), "labels": labels.pin_memory()}

        def step(batch):
            labels = batch["labels"]
            n_tokens = (labels != loss_fn.ignore_index).sum()
            out = model(batch["tokens"])
            loss = loss_fn(out, labels) * n_tokens
            loss.backward()
            if world > 1:
                dist.all_reduce(n_tokens)
                dist.all_reduce(loss)
            training.scale_grads_(model.parameters(), world / n_tokens)
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
            return loss.detach() / n_tokens

    def upload(h):
        return {k: v.to(device, non_blocking=True) for k, v in h.items()}

    hosts = [host_batch(1000 * rank + i) for i in range(4)]
    devs = [upload(h) for h in hosts]
    for i in range(args.warmup):
        step(devs[i % 4])
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    losses = []
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step(devs[i % 4])), args.steps)
    t_e2e = timed_loop(torch, dist, world, lambda i: losses.append(float(step(upload(hosts[i % 4])).item())), args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    tokens_per_step = hosts[0]["tokens"].numel() * world
    h2d = sum(t.numel() * t.element_size() for t in hosts[0].values())
    value = tokens_per_step * args.steps / t_kernel
    out = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_kernel / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "reference",
        "config": {
            "model": f"llama3_1_8b {'LoRA-DPO' if variant == 'dpo' else 'LoRA'} r64 alpha128 on q,k,v,o + w1,w2,w3",
            "global_batch": batch_per_gpu * world, "seq_len": dpo_len if variant == "dpo" else seq_len,
            "per_gpu_tokens": f"{2 * batch_per_gpu} x {dpo_len}" if variant == "dpo" else f"{batch_per_gpu} x {seq_len}",
            "parallelism": f"fsdp{world}" if world > 1 else "single", "activation_checkpointing": True,
            "optimizer": "torch.optim.AdamW fused lr 2e-5",
            "l2": "inputs larger than L2 (the base weights are streamed every step)",
        },
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": 0,
        "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2),
        "final_loss": float(losses[-1]) if losses else None,
    }
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_tensor_parallel(args, name, spec, lr, ClockSampler, timed_loop, dist_env) -> dict:
    """``bench.py --config 70b_tp8 | 70b_tp4dp2 --impl reference``: the reference's tensor-parallel full fine-tune
    (recipes/full_finetune_distributed.py:630-720): meta-device model → ``prepare_mha_for_tp`` → ``parallelize_module`` with
    ``base_llama_tp_plan`` (output projection patched by the loss for loss-parallel) → activation checkpointing → FSDP2 over the
    data-parallel mesh when it has more than one rank → activation offloading → fused AdamW."""
    if spec["family"] != "llama3_1":
        return {"impl": "reference", "unavailable": "the reference has no expert parallelism; only its Llama tensor-parallel configurations have an arm here"}
    try:
        _import_reference()
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference cannot be imported: {type(exc).__name__}: {exc}"[:300]}

    import torch
    import torch.distributed as dist
    from torch.distributed.tensor.parallel import parallelize_module
    from torchtune import modules, training
    from torchtune.models.llama3 import base_llama_tp_plan
    from torchtune.models.llama3_1 import llama3_1
    from torchtune.modules.attention_utils import packed_block_causal_mask
    from torchtune.modules.loss import LinearCrossEntropyLoss

    rank, world, local = dist_env()
    tp = min(spec["tp"], world)
    if world < 2 or world % tp:
        return {"impl": "reference", "unavailable": f"--config {name} needs a multiple of {tp} GPUs"}
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1234)
    dims = training.ParallelDims(dp_replicate=1, dp_shard=-1, tp=tp, cp=1, world_size=world)
    mesh = dims.build_mesh(device_type="cuda")
    dp_size = world // tp
    dp_rank = mesh["dp"].get_local_rank() if dims.dp_enabled else 0

    model_cfg = dict(spec["model"])
    if args.debug_layers:
        model_cfg["num_layers"] = args.debug_layers
    with training.set_default_dtype(torch.bfloat16), torch.device("meta"):
        model = llama3_1(**model_cfg)
    loss_fn = LinearCrossEntropyLoss()
    model = training.prepare_mha_for_tp(model, mesh["tp"])
    plan = base_llama_tp_plan(model)
    loss_fn.tp_enabled = True
    plan = loss_fn.patch_tp_plan(plan)
    parallelize_module(model, mesh["tp"], parallelize_plan=plan)
    training.set_activation_checkpointing(model, auto_wrap_policy={modules.TransformerSelfAttentionLayer})
    if dims.dp_shard_enabled:
        conditions = [partial(training.get_shard_conditions, names_to_match=["tok_embeddings", "output"])]
        training.shard_model(model=model, shard_conditions=conditions, cpu_offload=False, reshard_after_forward=True, dp_mesh=mesh["dp_shard_cp"])
    model.to_empty(device=device)
    with torch.no_grad():
        for p_ in model.parameters():
            if p_.dim() > 1:
                torch.nn.init.normal_(p_, std=0.02)
            else:
                p_.fill_(1.0)
        for m in model.modules():
            if hasattr(m, "rope_init"):
                with device:
                    m.rope_init()
    loss_fn.set_model_output(model)
    optimizer = torch.optim.AdamW(model.parameters(), lr=lr, fused=True)
    offload = bool(spec["offload"]) and not getattr(args, "ref_no_offload", False)
    offload_ctx = training.get_act_offloading_ctx_manager(model, offload)
    train_context = training.get_train_context(enable_loss_parallel=True)

    seq_len, doc_len, batch = spec["seq"], spec["doc"], spec["batch"]
    n_docs = seq_len // doc_len

    def host_batch(seed):
        g = torch.Generator().manual_seed(seed)
        tokens = torch.randint(0, model_cfg["vocab_size"], (batch, seq_len), generator=g, dtype=torch.long)
        labels = torch.roll(tokens, -1, dims=1)
        labels[:, doc_len - 1 :: doc_len] = -100
        pos = torch.arange(doc_len).repeat(n_docs).unsqueeze(0).expand(batch, seq_len).contiguous()
        seq_lens = torch.full((batch, n_docs), doc_len, dtype=torch.long)
        return {"tokens": tokens.pin_memory(), "labels": labels.pin_memory(), "input_pos": pos.pin_memory(), "seq_lens": seq_lens.pin_memory()}

    def upload(h):
        d = {k: v.to(device, non_blocking=True) for k, v in h.items()}
        d["mask"] = packed_block_causal_mask([row for row in d.pop("seq_lens")])
        return d

    def step(batch_):
        batch_ = dict(batch_)
        with train_context():
            labels = batch_.pop("labels")
            n_tokens = (labels != loss_fn.ignore_index).sum()
            with offload_ctx:
                out = model(**batch_)
            loss = loss_fn(out, labels) * n_tokens
            loss.backward()
        dist.all_reduce(n_tokens)
        dist.all_reduce(loss)
        training.scale_grads_(list(model.parameters()), world / n_tokens, False)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss.detach() / n_tokens

    hosts = [host_batch(1000 * dp_rank + i) for i in range(4)]
    devs = [upload(h) for h in hosts]
    for i in range(args.warmup):
        step(devs[i % 4])
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    losses = []
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step(devs[i % 4])), args.steps)
    t_e2e = timed_loop(torch, dist, world, lambda i: losses.append(float(step(upload(hosts[i % 4])).item())), args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    tokens_per_step = batch * seq_len * dp_size
    h2d = sum(t.numel() * t.element_size() for t in hosts[0].values())
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=device)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    value = tokens_per_step * args.steps / t_kernel
    out = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_kernel / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "reference",
        "config": {"model": spec["label"], "bench_config": name, "global_batch": batch * dp_size, "seq_len": seq_len, "doc_len": doc_len,
                   "parallelism": f"tp{tp}" + (f" x fsdp{dp_size}" if dp_size > 1 else "") + " (DTensor, sequence parallel norms, loss parallel)",
                   "activation_checkpointing": True, "activation_offloading": offload, "optimizer": "torch.optim.AdamW fused lr 2e-5",
                   "l2": "inputs larger than L2 (tens of GB of weights streamed every step)",
                   **({"debug_layers": args.debug_layers, "invalid": "reduced layer count: a functional check, not a benchmark number"} if args.debug_layers else {})},
        "clocks": clocks, "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": 0, "peak_mem_gib": round(float(peak.item()), 2), "final_loss": float(losses[-1]) if losses else None,
    }
    dist.destroy_process_group()
    return out if rank == 0 else {}
