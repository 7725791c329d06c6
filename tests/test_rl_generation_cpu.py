"""Rollout generation: optional logits and a stop-token exit that all ranks of a job agree on."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from torchtune_b200 import generation
from torchtune_b200.dev.rl.generation import generate as rl_generate
from torchtune_b200.models.llama2 import llama2


def _tiny():
    torch.manual_seed(0)
    return llama2(vocab_size=97, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=64, intermediate_dim=64).eval()


def test_without_logits_the_tokens_are_unchanged():
    model = _tiny()
    prompt = torch.randint(1, 97, (2, 5))
    ref, logits = generation.generate(model, prompt, max_generated_tokens=6, top_k=1, temperature=1e-6)
    out, none = rl_generate(model, prompt, max_generated_tokens=6, top_k=1, temperature=1e-6, return_logits=False)
    assert none is None and logits.shape == (2, 6, 97)
    assert torch.equal(out, ref)
    from torchtune_b200.dev.grpo.generation import generate as grpo_generate

    assert grpo_generate is rl_generate


def _rank(rank: int, port: int, out) -> None:
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=2)
    try:
        model = _tiny()
        torch.manual_seed(7)
        prompt = torch.randint(1, 97, (1, 4))
        free, _ = generation.generate(model, prompt, max_generated_tokens=8, top_k=1, temperature=1e-6)
        # rank 0 stops at its second generated token; rank 1 is given a token it never produces
        produced = set(free[0, 4:].tolist())
        stop = int(free[0, 5]) if rank == 0 else next(t for t in range(1, 97) if t not in produced)
        alone, _ = generation.generate(model, prompt, max_generated_tokens=8, top_k=1, temperature=1e-6, stop_tokens=[stop])
        together, _ = rl_generate(model, prompt, max_generated_tokens=8, top_k=1, temperature=1e-6, stop_tokens=[stop])
        out.put((rank, alone.shape[1], together.shape[1], together[0].tolist(), stop))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_ranks_stop_together():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        item = out.get(timeout=120)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    alone0, together0, tokens0, stop0 = got[0]
    alone1, together1, _, _ = got[1]
    assert alone0 < alone1 == 12  # on its own, rank 0 leaves the loop early
    assert together0 == together1 == 12  # as a group, nobody leaves before the slowest rank
    first = tokens0[4:].index(stop0)
    assert all(t == 0 for t in tokens0[4 + first + 1 :])  # rank 0's extra steps are padding
