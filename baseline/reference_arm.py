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
