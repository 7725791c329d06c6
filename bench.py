"""Headline benchmark: Llama-3.1-8B full fine-tune step throughput (tokens/s, whole job).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Config (fixed by the baseline definition): 32 layers, dim 4096, 32 heads / 8 KV heads, FFN
14336, vocab 128256, llama3 RoPE scaling; packed sequences of 2048 tokens with document
boundaries every 512 tokens (block-causal mask), per-GPU batch 4, activation checkpointing
on, AdamW lr 2e-5, bf16; synthetic uniform tokens and random-init weights.  Data parallel
over N GPUs with sharded optimizer state and fp32 gradient reduction (weak scaling: the
per-GPU batch is fixed).

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events, max over ranks)
with device-resident inputs; ``e2e`` times the public ``TrainStep`` call including the
pinned host→device input copy and the device→host loss read every step.
``--impl reference`` runs the unmodified reference implementation installed under
``baseline/_ref`` on the same config and prints the same line with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = dict(vocab_size=128_256, num_layers=32, num_heads=32, num_kv_heads=8, embed_dim=4096, max_seq_len=8192, intermediate_dim=14336, norm_eps=1e-5, rope_base=500_000)
SEQ_LEN, DOC_LEN, BATCH_PER_GPU, LR = 2048, 512, 4, 2e-5
BASELINE_TOKENS_PER_S = None  # the reference publishes no B200 number for this config

# The other benchmark configurations (``--config``); the default above stays the headline.
MODEL_70B = dict(vocab_size=128_256, num_layers=80, num_heads=64, num_kv_heads=8, embed_dim=8192, max_seq_len=8192, intermediate_dim=28672, norm_eps=1e-5, rope_base=500_000)
MODEL_SCOUT = dict(vocab_size=202_048, num_layers=48, num_heads=40, num_kv_heads=8, embed_dim=5120, hidden_dim=8192, max_seq_len=8192, rope_base=500_000, norm_eps=1e-5, num_experts=16,
                   use_shared_expert=True, skip_rope_interval=4, attention_chunk_size=8192, use_scaled_rope=True)
SHARDED_CONFIGS = {
    # name: model, builder, tensor-parallel size (0 = none), expert-parallel size, seq, doc length, batch per data-parallel rank, activation offload
    "70b_tp8": dict(model=MODEL_70B, family="llama3_1", tp=8, ep=0, seq=4096, doc=4096, batch=1, offload=True, label="llama3_3_70b"),
    "70b_tp4dp2": dict(model=MODEL_70B, family="llama3_1", tp=4, ep=0, seq=4096, doc=4096, batch=1, offload=True, label="llama3_3_70b"),
    "scout_ep8": dict(model=MODEL_SCOUT, family="llama4", tp=0, ep=8, seq=2048, doc=2048, batch=2, offload=False, label="llama4_scout_17b_16e (text decoder)"),
}


class ClockSampler:
    """Polls nvidia-smi during the timed region (SM clock, throttle reasons)."""

    QUERY = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
            return
        # nvidia-smi needs a moment to attach to the driver; during that time kernel launches of this process can stall.  The timed
        # region starts only once the first sample has arrived (the device is idle here: the caller has just synchronised), and the
        # samples taken before that are dropped.
        deadline = time.time() + 15.0
        while not self.rows and time.time() < deadline and self.proc.poll() is None:
            time.sleep(0.02)
        self.rows.clear()

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def synthetic_batch(torch, batch: int, seed: int, vocab: int = MODEL["vocab_size"], seq_len: int = SEQ_LEN, doc_len: int = DOC_LEN):
    """Host-side (pinned) packed batch: uniform tokens, shifted labels, per-document positions."""
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, vocab, (batch, seq_len), generator=g, dtype=torch.long)
    labels = torch.roll(tokens, -1, dims=1)
    labels[:, doc_len - 1 :: doc_len] = -100
    n_docs = seq_len // doc_len
    pos = torch.arange(doc_len).repeat(n_docs).unsqueeze(0).expand(batch, seq_len).contiguous()
    doc_ids = torch.arange(n_docs, dtype=torch.int32).repeat_interleave(doc_len).unsqueeze(0).expand(batch, seq_len).contiguous()
    pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
    return {"tokens": pin(tokens), "labels": pin(labels), "input_pos": pin(pos), "doc_ids": pin(doc_ids)}


def dist_env():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    return rank, world, local


def timed_loop(torch, dist, world, fn, steps: int):
    """Barrier + sync on both sides, CUDA events, max over ranks → seconds."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []
    e0.record()
    for i in range(steps):
        fn(i)
        if os.environ.get("TTB_BENCH_TRACE"):
            m = torch.cuda.Event(enable_timing=True)
            m.record()
            marks.append(m)
    e1.record()
    torch.cuda.synchronize()
    if marks and int(os.environ.get("RANK", "0")) == 0:
        prev, per_step = e0, []
        for m in marks:
            per_step.append(round(prev.elapsed_time(m), 1))
            prev = m
        print(f"[trace] per-step ms: {per_step}", file=sys.stderr, flush=True)
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / 1e3], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from torchtune_b200 import training
    from torchtune_b200.engine.train_step import TrainStep
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss
    from torchtune_b200.ops._lib import check_device_errors, lib
    from torchtune_b200.ops.mask import AttentionMask
    from torchtune_b200.optim import AdamW

    os.environ.setdefault("TTB_STRICT", "1")  # a bf16 CUDA op that would leave the sm_100a kernels raises instead of falling back
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    from torchtune_b200 import parallel as par

    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    # Engine: with more than one GPU the headline runs on the ZeRO-3 engine (every parameter, gradient and moment sharded, which is
    # what the reference's FSDP2 arm does): it measured within 1.5 % of the resident engine at 2, 4 and 8 GPUs with 0.29 - 0.6 x the
    # memory.  `--variant resident` forces whole parameters and gradients on every GPU, `--variant zero3` forces sharding at N = 1.
    zero3 = args.variant == "zero3" or (args.variant == "full" and world > 1 and not args.fp8)
    if zero3:
        from torchtune_b200.parallel.zero3 import Zero3Engine

        parallel = Zero3Engine(device)
    else:
        parallel = par.DataParallelEngine(device=device)  # world 1: same flat store, no peers
    torch.manual_seed(1234)  # identical initial weights on every rank
    with training.set_default_dtype(torch.bfloat16), (torch.device("meta") if zero3 else device):
        model = llama3_1(**MODEL)
        for name, p in model.named_parameters():
            if p.dim() > 1 and p.is_floating_point() and not p.is_meta:
                torch.nn.init.normal_(p, std=0.02)
    if args.fp8:  # optional variant, never the default: decoder linears (not the output head) on the fp8 tensor cores
        training.convert_to_float8_training(model, args.fp8_recipe)
    training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
    loss_fn = LinearCrossEntropyLoss(num_output_chunks=8)
    loss_fn.set_model_output(model)
    # zero3: the model is still on the meta device; every layer is given normal(0, 0.02) values right before it is cut into shards
    model = parallel.prepare(model, training.LayerwisePreparer(device)) if zero3 else parallel.prepare(model)
    optimizer = parallel.build_optimizer(model, lr=LR)
    step = TrainStep(model, loss_fn, optimizer, device, parallel=parallel)

    def to_model_batch(host):
        dev = step.upload(host)
        dev["mask"] = AttentionMask(causal=True, doc_ids=dev.pop("doc_ids"))
        return dev

    host_batches = [synthetic_batch(torch, BATCH_PER_GPU, seed=1000 * rank + i) for i in range(4)]
    dev_batches = [to_model_batch(h) for h in host_batches]
    tokens_per_step = BATCH_PER_GPU * SEQ_LEN * world
    L = lib()

    losses = []
    for i in range(args.warmup):
        losses.append(step.compute(dev_batches[i % 4]))
    torch.cuda.synchronize()
    check_device_errors()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ttb_launch_count()
    if os.environ.get("TTB_BENCH_TRACE"):
        step.trace_events = []
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step.compute(dev_batches[i % 4])), args.steps)
    if step.trace_events:
        ev, step.trace_events = step.trace_events, None
        per = len(ev) // args.steps
        names = ["fwd+loss", "bwd", "count", "optimizer"]
        sums = [0.0] * (per - 1)
        for k in range(args.steps):
            seg = ev[k * per : (k + 1) * per]
            phases = [round(a.elapsed_time(b), 1) for a, b in zip(seg[:-1], seg[1:])]
            sums = [x + y for x, y in zip(sums, phases)]
            if rank == 0 and sum(phases) > 1.15 * 1e3 * t_kernel / args.steps:
                print(f"[trace] slow step {k}: {dict(zip(names, phases))}", file=sys.stderr, flush=True)
        if rank == 0:
            print(f"[trace] mean phase ms: {dict(zip(names, [round(x / args.steps, 1) for x in sums]))}", file=sys.stderr, flush=True)
    launches = L.ttb_launch_count() - launches0

    def e2e_step(i):
        host = host_batches[i % 4]
        dev = to_model_batch(host)  # pinned host -> device copy of this step's inputs
        losses.append(float(step.compute(dev).item()))  # device -> host read of the loss

    t_e2e = timed_loop(torch, dist, world, e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    check_device_errors()
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0].values())
    peak_gib = (torch.cuda.max_memory_allocated() + par.PeerBuffer.peak_bytes) / 2**30  # torch's allocator + cudaMalloc'ed peer buffers
    final_loss = float(losses[-1]) if losses else float("nan")
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
        "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": ("fp8 linears (e4m3 values, one power-of-two scale per 32 values along each contraction, applied in the tensor core), bf16 elsewhere" if args.fp8_recipe == "blockwise"
                  else "fp8 linears (e4m3 / e5m2 operands, dynamic tensorwise scales), bf16 elsewhere") if args.fp8 else "bf16",
        "data": "synthetic uniform tokens, random-init weights",
        "impl": "ours",
        "config": {
            "model": "llama3_1_8b",
            "global_batch": BATCH_PER_GPU * world,
            "seq_len": SEQ_LEN,
            "doc_len": DOC_LEN,
            "parallelism": (f"zero3 x{world} (parameters, gradients and moments sharded; per-layer peer-memory gather)" if zero3 else f"dp{world}") if world > 1 else "single",
            "activation_checkpointing": True,
            "optimizer": "AdamW lr 2e-5, fused reduce-scatter+update kernel per layer during backward" if zero3 else "AdamW lr 2e-5, fused reduce+update+broadcast kernel over flat peer buffers",
            "l2": "inputs larger than L2 (16 GB of weights streamed every step)",
        },
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches),
        "peak_mem_gib": round(peak_gib, 2),
        "final_loss": final_loss,
    }
    if zero3:
        parallel.shutdown()
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


PEFT_BATCH_PER_GPU = 8  # adapter fine-tuning configurations: 8 sequences of 2048 (LoRA / QLoRA), 8 preference pairs of 2 x 1024 (DPO)
DPO_LEN, DPO_PROMPT, DPO_BETA = 1024, 256, 0.1


def peft_host_batch(torch, variant: str, seed: int, vocab: int = MODEL["vocab_size"]):
    """Pinned host batch of the adapter configurations.  ``lora`` / ``qlora``: 8 unpacked causal sequences of 2048 tokens.
    ``dpo``: 8 chosen then 8 rejected sequences of 1024 tokens; each pair shares its first 256 tokens (the prompt), whose labels
    are masked."""
    g = torch.Generator().manual_seed(seed)
    pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
    if variant == "dpo":
        prompt = torch.randint(0, vocab, (PEFT_BATCH_PER_GPU, DPO_PROMPT), generator=g, dtype=torch.long)
        tails = torch.randint(0, vocab, (2 * PEFT_BATCH_PER_GPU, DPO_LEN - DPO_PROMPT), generator=g, dtype=torch.long)
        tokens = torch.cat([torch.cat([prompt, prompt]), tails], dim=1)
        labels = tokens.clone()
        labels[:, :DPO_PROMPT] = -100
        return {"tokens": pin(tokens), "labels": pin(labels)}
    tokens = torch.randint(0, vocab, (PEFT_BATCH_PER_GPU, SEQ_LEN), generator=g, dtype=torch.long)
    labels = torch.roll(tokens, -1, dims=1)
    labels[:, -1] = -100
    return {"tokens": pin(tokens), "labels": pin(labels)}


def run_ours_peft(args) -> dict:
    """Adapter fine-tuning configurations (``--variant lora | qlora | dpo``): Llama-3.1-8B with LoRA r=64 / alpha=128 on the q, k,
    v, output projections and the MLP, frozen bf16 (``qlora``: NF4) base weights, per-GPU batch 8, data parallel over all ranks.
    ``dpo`` trains the adapters with the DPO loss (beta 0.1); its reference log-probabilities come from the same model with the
    adapters switched off, computed inside the timed step."""
    import torch
    import torch.distributed as dist

    from torchtune_b200 import parallel as par
    from torchtune_b200 import training
    from torchtune_b200.engine.preference import PreferenceStep
    from torchtune_b200.engine.train_step import TrainStep
    from torchtune_b200.models.llama3_1 import lora_llama3_1_8b
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss
    from torchtune_b200.modules.peft import get_adapter_params, set_trainable_params
    from torchtune_b200.ops._lib import check_device_errors, lib
    from torchtune_b200.rlhf.loss import DPOLoss

    os.environ.setdefault("TTB_STRICT", "1")
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    parallel = par.DataParallelEngine(device=device)
    torch.manual_seed(1234)
    with training.set_default_dtype(torch.bfloat16), device:
        model = lora_llama3_1_8b(lora_attn_modules=["q_proj", "k_proj", "v_proj", "output_proj"], apply_lora_to_mlp=True, lora_rank=64, lora_alpha=128,
                                 quantize_base=args.variant == "qlora")
        for name, p in model.named_parameters():
            if p.dim() > 1 and p.is_floating_point() and "lora_b" not in name:
                torch.nn.init.normal_(p, std=0.02)
    set_trainable_params(model, get_adapter_params(model))
    training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
    model = parallel.prepare(model)
    optimizer = parallel.build_optimizer(model, lr=LR)
    if args.variant == "dpo":
        step = PreferenceStep(model, DPOLoss(beta=DPO_BETA), optimizer, device, parallel=parallel)
    else:
        loss_fn = LinearCrossEntropyLoss(num_output_chunks=8)
        loss_fn.set_model_output(model)
        step = TrainStep(model, loss_fn, optimizer, device, parallel=parallel)

    host_batches = [peft_host_batch(torch, args.variant, seed=1000 * rank + i) for i in range(4)]
    dev_batches = [step.upload(h) for h in host_batches]
    tokens_per_step = host_batches[0]["tokens"].numel() * world  # every token of the batch, as both reference recipes count them
    L = lib()
    losses = []
    for i in range(args.warmup):
        losses.append(step.compute(dev_batches[i % 4]))
    torch.cuda.synchronize()
    check_device_errors()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ttb_launch_count()
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step.compute(dev_batches[i % 4])), args.steps)
    launches = L.ttb_launch_count() - launches0
    t_e2e = timed_loop(torch, dist, world, lambda i: losses.append(float(step(host_batches[i % 4]).item())), args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    check_device_errors()
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0].values())
    value = tokens_per_step * args.steps / t_kernel
    shape = f"{2 * PEFT_BATCH_PER_GPU} x {DPO_LEN} (8 pairs, shared {DPO_PROMPT}-token prompt)" if args.variant == "dpo" else f"{PEFT_BATCH_PER_GPU} x {SEQ_LEN}"
    out = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_kernel / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (NF4 base weights, block 64, double-quantised scales)" if args.variant == "qlora" else "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
        "config": {
            "model": f"llama3_1_8b {'LoRA-DPO' if args.variant == 'dpo' else ('QLoRA' if args.variant == 'qlora' else 'LoRA')} r64 alpha128 on q,k,v,o + w1,w2,w3",
            "global_batch": PEFT_BATCH_PER_GPU * world, "per_gpu_tokens": shape, "seq_len": DPO_LEN if args.variant == "dpo" else SEQ_LEN,
            "parallelism": f"dp{world}" if world > 1 else "single", "activation_checkpointing": True,
            "optimizer": "AdamW lr 2e-5 over the adapter parameters (fused reduce+update+broadcast kernel)",
            "l2": "inputs larger than L2 (the base weights are streamed every step)",
        },
        "clocks": clocks,
        "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches),
        "peak_mem_gib": round((torch.cuda.max_memory_allocated() + par.PeerBuffer.peak_bytes) / 2**30, 2),
        "final_loss": float(losses[-1]) if losses else float("nan"),
    }
    if args.variant == "dpo":
        out["config"]["loss"] = f"DPO beta {DPO_BETA}, reference = adapters disabled"
    parallel.shutdown()
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_ours_tp(args) -> dict:
    """Off-headline variant: the same model and batch shape with tensor + sequence parallelism over all ranks (every rank sees
    the same 4 × 2048 batch; fused all-gather → GEMM and GEMM → reduce-scatter kernels in every layer)."""
    import torch
    import torch.distributed as dist

    from torchtune_b200 import training
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss
    from torchtune_b200.ops._lib import check_device_errors, lib
    from torchtune_b200.ops.mask import AttentionMask
    from torchtune_b200.parallel.tp import TensorParallelContext
    from torchtune_b200.parallel.tp_model import tensor_parallelize

    rank, world, local = dist_env()
    if world < 2:
        return {"impl": "ours", "unavailable": "the tensor-parallel variant needs at least 2 GPUs"}
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(1234)
    with training.set_default_dtype(torch.bfloat16), device:
        model = llama3_1(**MODEL)
        for p in model.parameters():
            if p.dim() > 1:
                torch.nn.init.normal_(p, std=0.02)
    training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
    tp = TensorParallelContext(device, None, max_rows_per_rank=BATCH_PER_GPU * SEQ_LEN // world, max_width=MODEL["embed_dim"])
    model = tensor_parallelize(model, tp, activation_checkpointing=True)
    torch.cuda.empty_cache()
    loss_fn = LinearCrossEntropyLoss(num_output_chunks=8)
    loss_fn.set_model_output(model)
    optimizer = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=LR, fused=True)
    batches = []
    for i in range(4):
        host = synthetic_batch(torch, BATCH_PER_GPU, seed=i)  # identical on every rank
        dev = {k: v.to(device) for k, v in host.items()}
        dev["mask"] = AttentionMask(causal=True, doc_ids=dev.pop("doc_ids"))
        batches.append(dev)
    done = []

    def step(i):
        if len(done) >= 2:
            done.pop(0).synchronize()
        batch = dict(batches[i % 4])
        labels = model.shard_rows(batch.pop("labels"))
        loss_sum, n_valid = loss_fn.compute_sum(model(**batch), labels)
        loss_sum.backward()
        n = n_valid.to(torch.float32)
        dist.all_reduce(n)
        model.sync_replicated_grads()
        torch._foreach_mul_([p.grad for p in model.parameters() if p.grad is not None], (1.0 / n).to(torch.bfloat16))
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        ev = torch.cuda.Event()
        ev.record()
        done.append(ev)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    check_device_errors()
    L = lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ttb_launch_count()
    t = timed_loop(torch, dist, world, step, args.steps)
    launches = L.ttb_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    check_device_errors()
    tokens = BATCH_PER_GPU * SEQ_LEN
    out = {
        "metric": "tokens_per_second", "value": tokens * args.steps / t, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
        "config": {"model": "llama3_1_8b (tensor-parallel variant, not the headline)", "global_batch": BATCH_PER_GPU, "seq_len": SEQ_LEN, "doc_len": DOC_LEN,
                   "parallelism": f"tp{world} + sequence parallel", "activation_checkpointing": True, "optimizer": "torch.optim.AdamW fused on the shards"},
        "clocks": clocks, "gpu_launches": int(launches), "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2),
    }
    tp.close()
    dist.destroy_process_group()
    return out if rank == 0 else {}


def run_ours_sharded(args) -> dict:
    """``--config 70b_tp8 | 70b_tp4dp2 | scout_ep8``: whole training steps of the models that do not fit one GPU.

    The model is built on the meta device and given storage layer by layer while it is sliced (tensor parallel: fused
    all-gather → GEMM / GEMM → reduce-scatter kernels; expert parallel: peer-memory dispatch / combine + grouped GEMMs).  The
    optimizer is the fused pull-reduce → AdamW → push kernel over two flat stores (replicated parameters sharded over every
    rank, shards over their replicas), driven through the same public ``TrainStep`` as the headline."""
    import torch
    import torch.distributed as dist

    os.environ.setdefault("TTB_STRICT", "1")
    from torchtune_b200 import parallel as par
    from torchtune_b200 import training
    from torchtune_b200.engine.train_step import TrainStep
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss
    from torchtune_b200.ops._lib import check_device_errors, lib
    from torchtune_b200.ops.mask import AttentionMask

    spec = SHARDED_CONFIGS[args.config]
    rank, world, local = dist_env()
    tp = min(spec["tp"], world) if spec["tp"] else 1
    ep = min(spec["ep"], world) if spec["ep"] else 1
    if world < 2:
        return {"impl": "ours", "config": {"model": spec["label"]}, "unavailable": f"--config {args.config} needs at least 2 GPUs (the model does not fit one)"}
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    cfg = {"tensor_parallel_dim": tp, "expert_parallel_dim": ep, "batch_size": spec["batch"], "tensor_parallel_max_tokens": spec["batch"] * spec["seq"]}
    strategy = par.ParallelStrategy(cfg, device)
    model_kwargs = dict(spec["model"])
    if args.debug_layers:
        model_kwargs["num_layers"] = args.debug_layers
    with training.set_default_dtype(torch.bfloat16), torch.device("meta"):
        if spec["family"] == "llama4":
            from torchtune_b200.models.llama4 import llama4_decoder

            model = llama4_decoder(**model_kwargs)
        else:
            from torchtune_b200.models.llama3_1 import llama3_1

            model = llama3_1(**model_kwargs)
    training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
    model = strategy.shard_model(model, cfg, None)  # no checkpoint: normal(0, 0.02) weights, identical on every rank
    torch.cuda.empty_cache()
    loss_fn = LinearCrossEntropyLoss(num_output_chunks=8)
    loss_fn.set_model_output(model)
    optimizer = strategy.build_optimizer(model, {"_component_": "torch.optim.AdamW", "lr": LR})
    torch.cuda.empty_cache()
    offload = training.get_act_offloading_ctx_manager(model, True) if spec["offload"] else None
    step = TrainStep(model, loss_fn, optimizer, device, parallel=strategy, activations_ctx=offload)
    vocab, seq, doc, batch = model_kwargs["vocab_size"], spec["seq"], spec["doc"], spec["batch"]

    def to_model_batch(host):
        dev = step.upload(host)
        dev["mask"] = AttentionMask(causal=True, doc_ids=dev.pop("doc_ids")) if doc < seq else AttentionMask(causal=True)
        if doc >= seq:
            dev.pop("doc_ids", None)
        return dev

    # the ranks of one tensor-parallel group read the same batch; data-parallel (and expert-parallel) ranks read their own
    host_batches = [synthetic_batch(torch, batch, seed=1000 * strategy.dp_rank + i, vocab=vocab, seq_len=seq, doc_len=doc) for i in range(4)]
    dev_batches = [to_model_batch(h) for h in host_batches]
    tokens_per_step = batch * seq * strategy.dp_size
    L = lib()
    losses = []
    for i in range(args.warmup):
        losses.append(step.compute(dev_batches[i % 4]))
    torch.cuda.synchronize()
    check_device_errors()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.ttb_launch_count()
    t_kernel = timed_loop(torch, dist, world, lambda i: losses.append(step.compute(dev_batches[i % 4])), args.steps)
    launches = L.ttb_launch_count() - launches0

    def e2e_step(i):
        losses.append(float(step.compute(to_model_batch(host_batches[i % 4])).item()))

    t_e2e = timed_loop(torch, dist, world, e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    check_device_errors()
    extra = {}
    if ep > 1:
        from torchtune_b200.modules.moe import expert_load_imbalance

        imb = expert_load_imbalance(model)
        extra["expert_load_imbalance_max_over_mean"] = None if imb is None else round(float(imb), 3)
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0].values())
    peak = torch.tensor([(torch.cuda.max_memory_allocated() + par.PeerBuffer.peak_bytes) / 2**30], device=device)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    value = tokens_per_step * args.steps / t_kernel
    mode = f"tp{tp}" + (f" x dp{world // tp}" if world // tp > 1 else "") + " + sequence parallel" if tp > 1 else f"ep{ep}" + (f" x dp{world // ep}" if world // ep > 1 else "") + ", dense parameters replicated with optimizer state sharded over all ranks"
    out = {
        "metric": "tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_kernel / args.steps, "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
        "config": {"model": spec["label"], "bench_config": args.config, "global_batch": batch * strategy.dp_size, "seq_len": seq, "doc_len": doc, "parallelism": mode,
                   "activation_checkpointing": True, "activation_offloading": bool(spec["offload"]),
                   "optimizer": "AdamW lr 2e-5 (bf16 moments), fused reduce+update+broadcast kernel over two flat peer stores",
                   "l2": "inputs larger than L2 (tens of GB of weights streamed every step)", **({"debug_layers": args.debug_layers, "invalid": "reduced layer count: a functional check, not a benchmark number"} if args.debug_layers else {})},
        "clocks": clocks, "e2e": {"value": tokens_per_step * args.steps / t_e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches), "peak_mem_gib": round(float(peak.item()), 2), "final_loss": float(losses[-1]) if losses else float("nan"), **extra,
    }
    strategy.shutdown()
    return out if rank == 0 else {}


def run_reference(args) -> dict:
    from baseline.reference_arm import run as run_ref
    from baseline.reference_arm import run_peft

    if args.config != "8b":
        from baseline.reference_arm import run_tensor_parallel

        return run_tensor_parallel(args, args.config, SHARDED_CONFIGS[args.config], LR, ClockSampler, timed_loop, dist_env)
    if args.variant in ("zero3", "resident", "tp") or args.fp8:
        return {"impl": "reference", "unavailable": "the reference arm covers the full fine-tune (default), --variant lora | qlora | dpo and --config 70b_tp8 | 70b_tp4dp2"}
    if args.variant in ("lora", "qlora", "dpo"):
        return run_peft(args, MODEL, SEQ_LEN, PEFT_BATCH_PER_GPU, DPO_LEN, DPO_PROMPT, DPO_BETA, LR, ClockSampler, timed_loop, dist_env)
    return run_ref(args, MODEL, SEQ_LEN, DOC_LEN, BATCH_PER_GPU, LR, ClockSampler, timed_loop, dist_env)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--variant", choices=["full", "zero3", "resident", "lora", "qlora", "dpo", "tp"], default="full",
                    help="full: the headline full fine-tune (ZeRO-3 engine with more than one GPU, resident engine on one); zero3 / resident force an engine; lora / qlora / dpo: the adapter configurations at per-GPU batch 8; tp: tensor-parallel variant")
    ap.add_argument("--config", choices=["8b"] + sorted(SHARDED_CONFIGS), default="8b", help="8b: the headline (Llama-3.1-8B); the others are the 70B tensor-parallel and Scout expert-parallel configurations")
    ap.add_argument("--debug-layers", type=int, default=0, help="functional check of a --config on few GPUs: build only this many layers (the printed line is marked invalid)")
    ap.add_argument("--ref-no-offload", action="store_true", help="with --impl reference --config 70b_*: run the reference without its activation offloading (diagnostic)")
    ap.add_argument("--ref-compile", action="store_true", help="with --impl reference: the reference's `compile: True` path (informational; the default arm stays on the stock eager path)")
    ap.add_argument("--fp8-recipe", choices=["tensorwise", "blockwise"], default="tensorwise", help="with --fp8: one scale per tensor, or MX block scales (32 values per scale)")
    ap.add_argument("--fp8", action="store_true", help="variant: fp8 decoder linears (the headline number is always bf16)")
    args = ap.parse_args()
    rank, world, _ = dist_env()
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun when called directly with --gpus N
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", "29511", __file__, *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        result = run_reference(args)
    else:
        if args.config != "8b":
            result = run_ours_sharded(args)
        else:
            result = run_ours_tp(args) if args.variant == "tp" else (run_ours_peft(args) if args.variant in ("lora", "qlora", "dpo") else run_ours(args))
    if rank == 0:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
