"""bf16 CUDA paths of the MoE, vision and multimodal models against fp32 CPU-style references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from torchtune_b200 import ops


@pytest.fixture(autouse=True)
def _check_device_errors():
    yield
    if torch.cuda.is_available():
        from torchtune_b200.ops._lib import check_device_errors

        torch.cuda.synchronize()
        check_device_errors()


def _rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("T,K,N", [(256, 128, 192), (77, 64, 256), (1024, 512, 1024)])
def test_matmul_kn_forward_backward(T, K, N):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(T, K, generator=g, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(K, N, generator=g, device="cuda") * 0.1).bfloat16().requires_grad_()
    dy = (torch.randn(T, N, generator=g, device="cuda") * 0.2).bfloat16()
    y = ops.matmul(x, w)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf @ wf
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(w.grad, wf.grad) < 1e-2


def test_moe_layer_bf16_matches_fp32():
    from torchtune_b200.models.llama4 import llama4_moe

    torch.manual_seed(0)
    moe = llama4_moe(dim=256, hidden_dim=512, num_experts=8, experts_per_token=2).cuda()
    ref = llama4_moe(dim=256, hidden_dim=512, num_experts=8, experts_per_token=2).cuda()
    ref.load_state_dict(moe.state_dict())
    moe = moe.bfloat16()
    x = torch.randn(2, 96, 256, device="cuda") * 0.5
    xb = x.bfloat16().requires_grad_()
    y = moe(xb)
    y.float().sum().backward()
    with ops.use_reference_ops():
        # route with the bf16 model's choices so both sides evaluate the same experts
        xr = x.bfloat16().float().requires_grad_()
        for p, q in zip(ref.parameters(), moe.parameters()):
            p.data.copy_(q.data.float())
        yr = ref(xr)
        yr.sum().backward()
    assert _rel_err(y, yr) < 3e-2
    assert _rel_err(xb.grad, xr.grad) < 5e-2
    assert _rel_err(moe.experts.gate_proj.grad, ref.experts.gate_proj.grad) < 5e-2


def test_vision_encoder_bf16_matches_fp32():
    from torchtune_b200.models.clip import clip_vision_encoder

    torch.manual_seed(0)
    enc = clip_vision_encoder(tile_size=56, patch_size=14, embed_dim=128, num_layers=2, num_heads=4, max_num_tiles=4).cuda()
    images = torch.randn(2, 1, 4, 3, 56, 56, device="cuda")
    ar = torch.tensor([[[2, 2]], [[1, 3]]], device="cuda")
    with ops.use_reference_ops():
        want, _ = enc(images, ar)
    got, _ = enc.bfloat16()(images.bfloat16(), ar)
    assert got.shape == (2, 1, 4, 17, 128)
    assert _rel_err(got, want) < 3e-2


def test_llama4_tiny_train_step_bf16():
    from torchtune_b200.models.llama4 import llama4_decoder

    torch.manual_seed(0)
    model = llama4_decoder(vocab_size=512, num_layers=4, num_heads=4, num_kv_heads=2, embed_dim=256, hidden_dim=256, max_seq_len=256, num_experts=4, skip_rope_interval=2,
                           attention_chunk_size=64, use_scaled_rope=True).cuda().bfloat16()
    tokens = torch.randint(0, 512, (2, 128), device="cuda")
    logits = model(tokens)
    loss = F.cross_entropy(logits.float().reshape(-1, 512), tokens.reshape(-1))
    loss.backward()
    assert torch.isfinite(loss) and abs(loss.item() - 6.24) < 0.5  # ln 512
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
