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
    # Tokens route independently; keep only those whose top-k choice is the same under the bf16 and
    # the fp32 router, so both sides evaluate the same experts (a near-tie flips under bf16 rounding).
    flat = x.reshape(-1, 256)
    moe.router(flat.bfloat16())
    sel_b = moe.router.selected_experts_indices.sort(dim=1).values
    with ops.use_reference_ops():
        ref.bfloat16().float().router(flat.bfloat16().float())
    sel_f = ref.router.selected_experts_indices.sort(dim=1).values
    keep = (sel_b == sel_f).all(dim=1)
    assert keep.float().mean() > 0.8
    x = flat[keep][None]
    xb = x.bfloat16().requires_grad_()
    y = moe(xb)
    y.float().sum().backward()
    with ops.use_reference_ops():
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
    # head dim 64 (2 heads of a 128-wide encoder) keeps the attention on the sm_100a kernel, as the CLIP presets' 64 / 80-wide heads do not all do
    enc = clip_vision_encoder(tile_size=56, patch_size=14, embed_dim=128, num_layers=2, num_heads=2, max_num_tiles=4).cuda()
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


def test_llama3_1_bf16_on_native_kernels_matches_transformers_fp32():
    """The flagship architecture end to end on the sm_100a kernels (bf16, head dim 128, grouped-query attention, scaled rotary
    embedding) against the `transformers` implementation in fp32 on the same random weights."""
    transformers = pytest.importorskip("transformers")
    from torchtune_b200.models.convert_weights import hf_to_tune
    from torchtune_b200.models.llama3_1 import llama3_1

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                   max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False,
                                   rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192))
    hf = transformers.LlamaForCausalLM(cfg).eval().float().cuda()
    with torch.device("cuda"):
        mine = llama3_1(vocab_size=4096, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=512, max_seq_len=1024, intermediate_dim=1024, rope_base=500000, scale_factor=8)
    mine.load_state_dict(hf_to_tune({k: v for k, v in hf.state_dict().items()}, num_heads=4, num_kv_heads=2, dim=512))
    mine = mine.to(torch.bfloat16).eval()
    tokens = torch.randint(0, 4096, (2, 512), device="cuda")
    with torch.no_grad():
        want = hf(input_ids=tokens).logits
        got = mine(tokens)
    assert _rel_err(got, want) < 3e-2
    assert (got.float().argmax(-1) == want.argmax(-1)).float().mean() > 0.9


def test_gemma2_tiny_bf16_capped_loss_matches_capped_logits():
    """Gemma-2 on the native kernels (head dim 128, soft-capped attention scores, sliding window on even layers): the loss taken
    from the hidden states — soft cap inside the fused linear + cross-entropy kernel — equals cross entropy over the decoder's own
    capped logits, and so do the gradients."""
    from torchtune_b200.models.gemma2 import gemma2
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss

    torch.manual_seed(0)
    with torch.device("cuda"):
        model = gemma2(vocab_size=4096, num_layers=2, num_heads=4, head_dim=128, num_kv_heads=2, embed_dim=512, intermediate_dim=1024, max_seq_len=512,
                       hidden_capping_value=50.0, final_capping_value=30.0, sliding_window_size=128).to(torch.bfloat16)
    with torch.no_grad():
        model.tok_embeddings.weight.mul_(30.0)  # drives the logits onto the flat part of the tanh
    tokens = torch.randint(0, 4096, (2, 256), device="cuda")
    labels = torch.randint(0, 4096, (2, 256), device="cuda")
    labels[:, :5] = -100
    logits = model(tokens)
    assert float(logits.detach().abs().max()) <= 30.0 and float(logits.detach().abs().max()) > 25.0
    want = F.cross_entropy(logits.float().reshape(-1, 4096), labels.reshape(-1), ignore_index=-100)
    want.backward()
    want_grad = model.layers[0].mlp.w1.weight.grad.float().clone()
    model.zero_grad()
    loss_fn = LinearCrossEntropyLoss()
    loss_fn.set_model_output(model)
    assert loss_fn.logit_softcap == 30.0
    got = loss_fn(model(tokens), labels)
    got.backward()
    assert abs(got.item() - want.item()) < 2e-3 * abs(want.item())
    assert _rel_err(model.layers[0].mlp.w1.weight.grad, want_grad) < 2e-2


@pytest.mark.parametrize("rank,dropout_input", [(8, False), (64, True)])
def test_lora_linear_fused_matches_reference(rank, dropout_input):
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).bfloat16()
    x, w, a, b, bias = mk(2, 96, 256, sc=0.5), mk(384, 256, sc=0.05), mk(rank, 256, sc=0.05), mk(384, rank, sc=0.05), mk(384, sc=0.1)
    xd = (x * (torch.rand(x.shape, generator=g, device="cuda") > 0.1)).bfloat16() if dropout_input else x
    leaves = [t.clone().requires_grad_() for t in (x, w, a, b, bias)]
    xx, ww, aa, bb, bi = leaves
    y = ops.lora_linear(xx, xd if dropout_input else xx, ww, bi, aa, bb, 2.0)
    dy = mk(2, 96, 384, sc=0.2)
    y.backward(dy)
    ref = [t.detach().float().requires_grad_() for t in (x, w, a, b, bias)]
    xr, wr, ar, br, bir = ref
    xdr = xd.float() if dropout_input else xr
    yr = F.linear(xr, wr, bir) + 2.0 * F.linear(F.linear(xdr, ar), br)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    for name, got, want in zip("x w a b bias".split(), leaves, ref):
        assert _rel_err(got.grad, want.grad) < 3e-2, name


def test_nf4_dequant_kernel_matches_reference():
    from torchtune_b200.modules.low_precision.nf4 import NF4Weight
    from torchtune_b200.ops import reference as ref

    torch.manual_seed(0)
    w = torch.randn(512, 1024, device="cuda") * 0.05
    nf4 = NF4Weight(512, 1024, device="cuda")
    nf4.quantize_(w.bfloat16())
    got = nf4.dequantize(torch.bfloat16)
    want = ref.nf4_dequantize(nf4.weight_nf4, nf4.scaler_q, nf4.scaler_factor, nf4.scaler_mean, (512, 1024), 64, 256, torch.bfloat16)
    assert torch.equal(got, want)
    assert _rel_err(got, w) < 0.12  # 4-bit quantisation error


def test_qlora_linear_trains_on_gpu():
    from torchtune_b200.modules.peft import LoRALinear

    torch.manual_seed(0)
    with torch.device("cuda"):
        lin = LoRALinear(1024, 512, rank=16, alpha=32, quantize_base=True).bfloat16()
    x = (torch.randn(4, 64, 1024, device="cuda") * 0.5).bfloat16().requires_grad_()
    y = lin(x)
    y.float().pow(2).mean().backward()
    assert y.shape == (4, 64, 512) and x.grad is not None and lin.lora_b.weight.grad is not None
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()


@pytest.mark.parametrize("counts,K,N", [([128, 128, 128, 128], 192, 320), ([5, 0, 300, 77], 192, 320), ([0, 0, 0, 513], 192, 320), ([1, 1, 1, 1], 192, 320),
                                        ([700, 64, 0, 1, 333, 129, 63, 1000], 1024, 1536)])
def test_grouped_matmul_matches_loop(counts, K, N):
    g = torch.Generator(device="cuda").manual_seed(1)
    E = len(counts)
    rows = sum(counts)
    x = (torch.randn(rows, K, generator=g, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(E, K, N, generator=g, device="cuda") * 0.1).bfloat16().requires_grad_()
    cnt = torch.tensor(counts, device="cuda")
    y = ops.grouped_matmul(x, w, cnt)
    dy = (torch.randn(rows, N, generator=g, device="cuda") * 0.2).bfloat16()
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    outs, s = [], 0
    for e, n in enumerate(counts):
        outs.append(xf[s : s + n] @ wf[e])
        s += n
    yf = torch.cat(outs)
    yf.backward(dy.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(w.grad, wf.grad) < 2e-2


# ----------------------------------------------------------------------------- sharded-parameter (ZeRO-3) engine on one GPU
@pytest.mark.parametrize("mode", ["fused", "deferred"])
def test_zero3_engine_single_gpu_tracks_fp32_adamw(mode):
    """World size 1 runs every kernel of the engine (bucket gather into a released buffer, reduce → AdamW on the shard store, the
    deferred update after clipping) with nothing to wait for: three bf16 steps must follow an fp32 AdamW run, and no parameter
    may stay resident between steps."""
    from torchtune_b200 import training
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.parallel.zero3 import Zero3Engine

    arch = dict(vocab_size=512, num_layers=3, num_heads=4, num_kv_heads=2, embed_dim=256, max_seq_len=128, intermediate_dim=512)
    dev = torch.device("cuda")
    torch.manual_seed(0)
    ref = llama3_1(**arch).to(dev)
    for p in ref.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
    with training.set_default_dtype(torch.bfloat16), dev:
        model = llama3_1(**arch)
    model.load_state_dict({k: v.bfloat16() for k, v in ref.state_dict().items()})
    ref.load_state_dict({k: v.float() for k, v in model.state_dict().items()})  # same bf16-rounded starting point
    training.set_activation_checkpointing(model, {TransformerSelfAttentionLayer})
    engine = Zero3Engine(dev)
    model = engine.prepare(model)
    opt = engine.build_optimizer(model, lr=1e-3, weight_decay=0.01)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.01)
    clip = 1.0 if mode == "deferred" else None
    g = torch.Generator(device="cuda").manual_seed(1)
    for step in range(3):
        tokens = torch.randint(0, 512, (2, 128), generator=g, device=dev)
        labels = torch.randint(0, 512, (2, 128), generator=g, device=dev)
        loss = F.cross_entropy(model(tokens).float().reshape(-1, 512), labels.reshape(-1), reduction="sum")
        if mode == "fused":
            assert engine.arm_backward_overlap(opt, 1.0 / 256, None)
        loss.backward()
        norm = engine.optimizer_step(model, opt, 1.0 / 256, clip)
        want = F.cross_entropy(ref(tokens).reshape(-1, 512), labels.reshape(-1), reduction="sum")
        (want / 256).backward()
        if clip is not None:
            want_norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), clip)
            assert abs(float(norm) - float(want_norm)) / float(want_norm) < 3e-2
        ref_opt.step()
        ref_opt.zero_grad()
        assert abs(loss.item() - want.item()) / want.item() < 2e-2, (step, loss.item(), want.item())
        assert all(p.untyped_storage().size() == 0 for p in model.parameters())
    got = engine.full_state_dict(model)
    for k, v in ref.state_dict().items():
        assert _rel_err(got[k], v.cpu()) < 2e-2, k
    engine.shutdown()


def test_zero3_gather_kernel_emulated_ranks():
    """``ttb_zero3_gather`` with the shards of four ranks held in four buffers of one device (peer mappings on a real group)."""
    import ctypes

    from torchtune_b200.ops._lib import check, lib, stream_ptr
    from torchtune_b200.parallel.dp import _declare_dp

    L = lib()
    _declare_dp(L)
    world, piece = 4, 8 * 1031
    shards = [torch.randn(piece, device="cuda").bfloat16() for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in shards])
    for rank in range(world):
        for ctas in (0, 3):
            dst = torch.zeros(world * piece, dtype=torch.bfloat16, device="cuda")
            check(L.ttb_zero3_gather(ptrs, world, rank, piece, dst.data_ptr(), None, 0, 0, None, ctas, stream_ptr()), "gather")
            assert torch.equal(dst, torch.cat(shards))
