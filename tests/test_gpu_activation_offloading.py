"""Activation offloading on a GPU: gradients with activations staged through pinned host memory (side stream or compute stream)
must equal the gradients of the plain run bit for bit, also when unrelated work keeps the compute stream busy between forward and
backward and when the pinned pool is recycled over several steps (the reference's stream-ordering cases:
tests/torchtune/training/test_activation_offloading.py:47-227)."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu

from torchtune_b200.training._activation_offloading import NoOpManager, OffloadActivations, get_act_offloading_ctx_manager


class _Net(nn.Module):
    def __init__(self, dim: int = 256, depth: int = 6):
        super().__init__()
        self.layers = nn.ModuleList([nn.Linear(dim, dim) for _ in range(depth)])
        self.output = nn.Linear(dim, 64)

    def forward(self, x):
        for layer in self.layers:
            x = x + torch.nn.functional.gelu(layer(x))
        return self.output(x)


def _grads(model, x, ctx, busy=False):
    model.zero_grad(set_to_none=True)
    with ctx:
        loss = model(x).float().pow(2).mean()
    if busy:  # unrelated kernels queued on the compute stream while the device→host copies are still in flight
        junk = torch.randn(2048, 2048, device="cuda")
        for _ in range(8):
            junk = junk @ junk * 1e-3
    loss.backward()
    torch.cuda.synchronize()
    return loss.detach().clone(), [p.grad.clone() for p in model.parameters()]


@pytest.mark.parametrize("use_streams", [True, False])
def test_offloaded_gradients_equal_resident_gradients(use_streams):
    torch.manual_seed(0)
    model = _Net().cuda().bfloat16()
    x = torch.randn(64, 128, 256, device="cuda", dtype=torch.bfloat16)
    import contextlib

    want_loss, want = _grads(model, x, contextlib.nullcontext())
    ctx = OffloadActivations(use_streams=use_streams, min_offload_size=1024)
    ctx.register_resident(model)
    for step in range(3):  # the pinned pool is recycled from the second step on
        loss, got = _grads(model, x, ctx, busy=(step == 1))
        assert torch.equal(loss, want_loss)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert ctx._next_id > 0, "nothing was offloaded"
    hosts = [s.host for s in ctx._slots.values() if s.host is not None]
    assert hosts and all(h.is_pinned() and not h.is_cuda for h in hosts)


def test_small_tensors_parameters_and_noop_regions_stay_on_the_device():
    torch.manual_seed(0)
    model = _Net(dim=64, depth=2).cuda()
    ctx = OffloadActivations(min_offload_size=1 << 30)  # nothing is large enough
    ctx.register_resident(model)
    x = torch.randn(4, 8, 64, device="cuda")
    with ctx:
        model(x).sum().backward()
    assert ctx._next_id == 0
    ctx = OffloadActivations(min_offload_size=16)
    ctx.register_resident(model)
    with ctx, NoOpManager():  # an inner no-op region switches offloading off
        model(x).sum().backward()
    assert ctx._next_id == 0


def test_recipe_context_exempts_the_output_projection():
    torch.manual_seed(0)
    model = _Net().cuda().bfloat16()
    x = torch.randn(8, 128, 256, device="cuda", dtype=torch.bfloat16)
    import contextlib

    want_loss, want = _grads(model, x, contextlib.nullcontext())
    ctx = get_act_offloading_ctx_manager(model, enable_activation_offloading=True)
    loss, got = _grads(model, x, ctx)
    assert torch.equal(loss, want_loss) and all(torch.equal(a, b) for a, b in zip(got, want))
    out_in_bytes = 8 * 128 * 256 * 2
    assert all(s.host is None or s.host.numel() * s.host.element_size() >= 1024 for s in ctx._slots.values())
    assert ctx._next_id >= len(model.layers) and out_in_bytes > 0
    assert isinstance(get_act_offloading_ctx_manager(model, enable_activation_offloading=False), contextlib.nullcontext)
