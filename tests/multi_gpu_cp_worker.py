"""Worker for the 2-GPU context-parallel exchange check: the head / sequence exchange as a push over peer memory against the
collective-library all-to-all, forward and backward, repeated so that the "buffer free" / "data arrived" flags cycle, with a
larger tensor in between so that the receive buffer is replaced once."""
import os

import torch
import torch.distributed as dist


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()

    from torchtune_b200.ops._lib import check_device_errors
    from torchtune_b200.parallel.cp import ContextParallelContext

    peer = ContextParallelContext(None)
    plain = ContextParallelContext(None)
    os.environ["TTB_CP_PEER"] = "1"

    def both(fn_name, x):
        os.environ["TTB_CP_PEER"] = "1"
        a = x.detach().clone().requires_grad_()
        ya = getattr(peer, fn_name)(a)
        g = torch.randn(ya.shape, generator=torch.Generator(device=dev).manual_seed(7 + rank), device=dev).to(x.dtype)
        ya.backward(g)
        os.environ["TTB_CP_PEER"] = "0"
        b = x.detach().clone().requires_grad_()
        yb = getattr(plain, fn_name)(b)
        yb.backward(g)
        assert torch.equal(ya, yb), (fn_name, tuple(x.shape))
        assert torch.equal(a.grad, b.grad), (fn_name, tuple(x.shape), "grad")
        return ya.detach()

    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    for it, (b, s_l, h, d) in enumerate([(2, 64, 8, 64), (1, 128, 4, 128), (2, 512, 16, 128), (2, 64, 8, 64), (3, 32, 2, 16)]):
        x = torch.randn(b, s_l, h, d, generator=gen, device=dev).bfloat16()
        y = both("seq_to_heads", x)
        assert y.shape == (b, s_l * world, h // world, d)
        back = both("heads_to_seq", y)
        assert torch.equal(back, x)  # the two exchanges are inverses
        kv = torch.randn(b, s_l, 1, d, generator=gen, device=dev).bfloat16()  # fewer K/V heads than ranks: heads are repeated
        both("seq_to_heads", kv)
    assert peer._peer is not None and peer._peer.epoch >= 20
    torch.cuda.synchronize()
    check_device_errors()
    peer.shutdown()
    dist.barrier()
    if rank == 0:
        print("CP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
