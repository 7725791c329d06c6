"""Numerics of every sm_100a kernel against a plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from torchtune_b200 import ops
from torchtune_b200.ops import reference as ref
from torchtune_b200.ops.mask import AttentionMask


@pytest.fixture(autouse=True)
def _check_device_errors():
    yield
    if torch.cuda.is_available():
        from torchtune_b200.ops._lib import check_device_errors

        torch.cuda.synchronize()
        check_device_errors()


def _rand(*shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


def _close(got, want, rtol, atol, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad}/{err.numel()} elements off, max err {err.max().item():.4g} (max ref {want.abs().max().item():.4g})"


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 256, 128), (200, 96, 320), (1024, 1024, 512), (384, 2048, 1088)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from torchtune_b200.ops._cuda import gemm

    a = _rand(M, K, seed=1)
    b = _rand(N, K, seed=2)
    want = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    got = gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn)
    _close(got, want, 2e-2, 2e-2 * math.sqrt(K) / 8, f"gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")


def test_gemm_epilogues():
    from torchtune_b200.ops._cuda import gemm

    a, b = _rand(512, 256, seed=3), _rand(384, 256, seed=4)
    bias = _rand(384, seed=5)
    want = a.float() @ b.float().t()
    _close(gemm(a, b, bias=bias), want + bias.float(), 2e-2, 0.1, "bias")
    out32 = gemm(a, b, out_dtype=torch.float32)
    _close(out32, want, 1e-3, 1e-2, "fp32 out")
    acc = out32.clone()
    gemm(a, b, out=acc, accumulate=True)
    _close(acc, 2 * want, 1e-3, 2e-2, "fp32 accumulate")
    accb = gemm(a, b)
    gemm(a, b, out=accb, accumulate=True, alpha=0.5)
    _close(accb, 1.5 * want, 3e-2, 0.2, "bf16 accumulate + alpha")


def test_gemm_large_matches_matmul():
    from torchtune_b200.ops._cuda import gemm

    a, b = _rand(4096, 4096, seed=6, scale=0.5), _rand(2048, 4096, seed=7, scale=0.5)
    want = torch.matmul(a, b.t())
    _close(gemm(a, b), want, 2e-2, 0.5, "large")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (520, 776, 136), (1000, 264, 72), (2304, 4352, 1088)])
def test_gemm_cta_pair_kernel(M, N, K, a_mn, b_mn):
    """``tcgen05.mma.cta_group::2`` kernel (two SMs per 256 × 256 tile) through its exported symbol: all four operand layouts,
    sizes that are not tile multiples, bias and bf16 accumulation into an existing output."""
    from torchtune_b200.ops._lib import check, check_device_errors, err_word, lib, stream_ptr

    a, b = _rand(M, K, seed=1), _rand(N, K, seed=2)
    bias, prev = _rand(N, seed=3), _rand(M, N, seed=4)
    want = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    L = lib()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    check(L.ttb_gemm_bf16_2sm(a_in.data_ptr(), b_in.data_ptr(), out.data_ptr(), M, N, K, int(a_mn), int(b_mn), a_in.stride(0), b_in.stride(0), N, 0, None, 1.0,
                              err_word(out.device).data_ptr(), stream_ptr()), "pair gemm")
    acc = prev.clone()
    check(L.ttb_gemm_bf16_2sm(a_in.data_ptr(), b_in.data_ptr(), acc.data_ptr(), M, N, K, int(a_mn), int(b_mn), a_in.stride(0), b_in.stride(0), N, 1, bias.data_ptr(), 0.5,
                              err_word(out.device).data_ptr(), stream_ptr()), "pair gemm accumulate")
    torch.cuda.synchronize()
    check_device_errors()
    tol = 2e-2 * math.sqrt(K) / 8
    _close(out, want, 2e-2, tol, f"pair gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")
    _close(acc, 0.5 * want + bias.float() + prev.float(), 3e-2, tol + 0.05, "pair gemm accumulate + bias + alpha")


def test_gemm_benchmark_shapes_match_matmul():
    """The projections of the benchmark model (4 × 2048 tokens, width 4096, MLP 14336) in the three GEMM forms of a step."""
    from torchtune_b200.ops._cuda import gemm

    x, w = _rand(8192, 4096, seed=21, scale=0.5), _rand(14336, 4096, seed=22, scale=0.05)
    y = gemm(x, w)  # forward
    _close(y, torch.matmul(x, w.t()), 2e-2, 0.3, "fwd 8192x14336x4096")
    dy = _rand(8192, 14336, seed=23, scale=0.1)
    _close(gemm(dy, w, b_mn=True), torch.matmul(dy, w), 2e-2, 0.3, "dgrad 8192x4096x14336")
    _close(gemm(dy, x, a_mn=True, b_mn=True), torch.matmul(dy.t(), x), 2e-2, 1.0, "wgrad 14336x4096x8192")


@pytest.mark.parametrize("n_out", [512, 4, 1])  # 4 and 1: output widths that are not a multiple of 8 (router over 4 experts, scalar head)
def test_linear_autograd(n_out):
    x = _rand(3, 40, 256, seed=8).requires_grad_()
    w = _rand(n_out, 256, seed=9, scale=0.05).requires_grad_()
    bias = _rand(n_out, seed=10).requires_grad_()
    y = ops.linear(x, w, bias)
    assert y.shape == (3, 40, n_out)
    gy = _rand(3, 40, n_out, seed=11)
    y.backward(gy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(gy.float())
    _close(y, yr, 2e-2, 5e-2, "linear fwd")
    _close(x.grad, xr.grad, 2e-2, 5e-2, "linear dx")
    _close(w.grad, wr.grad, 2e-2, 0.3, "linear dw")
    _close(bias.grad, br.grad, 2e-2, 0.3, "linear db")


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("rows,D", [(37, 256), (1024, 4096), (5, 8192), (19, 1536), (7, 12288), (2051, 2048)])
def test_rmsnorm(rows, D):
    x = _rand(rows, D, seed=1).requires_grad_()
    scale = (1 + 0.1 * _rand(D, seed=2).float()).to(torch.bfloat16).requires_grad_()
    y = ops.rms_norm(x, scale, 1e-5)
    gy = _rand(rows, D, seed=3)
    y.backward(gy)
    xr, sr = x.detach().float().requires_grad_(), scale.detach().float().requires_grad_()
    yr = ref.rms_norm(xr, sr, 1e-5)
    yr.backward(gy.float())
    _close(y, yr, 1e-2, 1e-2, "rmsnorm fwd")
    _close(x.grad, xr.grad, 2e-2, 2e-2, "rmsnorm dx")
    _close(scale.grad, sr.grad, 2e-2, 0.05 * math.sqrt(rows), "rmsnorm dscale")
    # weight-less variant
    y2 = ops.rms_norm(x.detach(), None, 1e-6)
    _close(y2, ref.rms_norm(x.detach().float(), None, 1e-6), 1e-2, 1e-2, "rmsnorm no scale")


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("use_pos", [False, True])
def test_rope(interleaved, use_pos):
    from torchtune_b200.modules import RotaryPositionalEmbeddings

    b, s, h, d = 2, 48, 4, 128
    rope = RotaryPositionalEmbeddings(d, max_seq_len=256, base=500000).cuda()
    x = _rand(b, s, h, d, seed=1).requires_grad_()
    pos = torch.randint(0, 256, (b, s), device="cuda") if use_pos else None
    y = ops.rope(x, rope.cache, pos, interleaved=interleaved)
    gy = _rand(b, s, h, d, seed=2)
    y.backward(gy)
    xr = x.detach().float().requires_grad_()
    fn = ref.rope_interleaved if interleaved else ref.rope_half
    yr = fn(xr, rope.cache, pos)
    yr.backward(gy.float())
    _close(y, yr, 1e-2, 1e-2, "rope fwd")
    _close(x.grad, xr.grad, 1e-2, 1e-2, "rope bwd")


def test_swiglu():
    g = _rand(70, 1536, seed=1).requires_grad_()
    u = _rand(70, 1536, seed=2).requires_grad_()
    y = ops.swiglu(g, u)
    gy = _rand(70, 1536, seed=3)
    y.backward(gy)
    gr, ur = g.detach().float().requires_grad_(), u.detach().float().requires_grad_()
    yr = ref.swiglu(gr, ur)
    yr.backward(gy.float())
    _close(y, yr, 2e-2, 2e-2, "swiglu fwd")
    _close(g.grad, gr.grad, 2e-2, 2e-2, "swiglu dg")
    _close(u.grad, ur.grad, 2e-2, 2e-2, "swiglu du")


# ------------------------------------------------------------------ loss
@pytest.mark.parametrize("T,D,V", [(300, 256, 1024), (1000, 512, 32000), (2048, 1024, 128256)])  # last: the benchmark model's vocabulary
def test_linear_cross_entropy(T, D, V):
    h = _rand(T, D, seed=1).requires_grad_()
    w = _rand(V, D, seed=2, scale=0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss, n = ops.linear_cross_entropy(h, w, labels, -100, 8)
    (loss / n).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr, nr = ref.linear_cross_entropy(hr, wr, labels, -100, 8)
    (lr / nr).backward()
    assert n.item() == nr.item()
    _close(loss / n, lr / nr, 5e-3, 5e-3, "ce loss")
    _close(h.grad, hr.grad, 5e-2, 2e-4, "ce dh")
    _close(w.grad, wr.grad, 5e-2, 2e-4, "ce dw")


@pytest.mark.parametrize("T,D,V,cap", [(300, 256, 1024, 2.0), (1000, 512, 32000, 30.0)])
def test_linear_cross_entropy_with_soft_capped_logits(T, D, V, cap):
    """Gemma-2: softmax over cap·tanh(logits/cap); the small cap puts most logits on the curved part of the tanh."""
    h = _rand(T, D, seed=1).requires_grad_()
    w = _rand(V, D, seed=2, scale=0.25).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss, n = ops.linear_cross_entropy(h, w, labels, -100, 8, softcap=cap)
    (loss / n).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr, nr = ref.linear_cross_entropy(hr, wr, labels, -100, 8, softcap=cap)
    (lr / nr).backward()
    assert n.item() == nr.item()
    uncapped, _ = ref.linear_cross_entropy(hr.detach(), wr.detach(), labels, -100, 8)
    assert abs((uncapped / nr - lr / nr).item()) > 1e-2  # the cap changes this loss, so the comparison below means something
    _close(loss / n, lr / nr, 5e-3, 5e-3, "capped ce loss")
    _close(h.grad, hr.grad, 5e-2, 3e-4, "capped ce dh")
    _close(w.grad, wr.grad, 5e-2, 3e-4, "capped ce dw")


@pytest.mark.parametrize("dtype,n", [(torch.bfloat16, 256 * 64), (torch.bfloat16, 1000 * 7), (torch.float32, 4096 + 8)])
def test_adamw8bit_kernel_matches_statement(dtype, n):
    """Five steps of the 8-bit-moment AdamW kernel against the PyTorch statement of the same arithmetic on the same inputs: codes may
    differ by one step where the fp32 rounding of a square root falls on a tie; parameters stay within bf16 / fp32 rounding."""
    from torchtune_b200.ops import _cuda

    torch.manual_seed(0)
    p0 = (torch.randn(n, device="cuda") * 0.1).to(dtype)
    state = lambda: (torch.zeros(n, dtype=torch.int8, device="cuda"), torch.zeros(n, dtype=torch.uint8, device="cuda"),
                     torch.zeros((n + 255) // 256, device="cuda"), torch.zeros((n + 255) // 256, device="cuda"))
    pk, (mq, vq, ms, vs) = p0.clone(), state()
    pr, (mqr, vqr, msr, vsr) = p0.clone().float(), state()
    scale = torch.tensor(0.5, device="cuda")
    for step in range(1, 6):
        g = (torch.randn(n, device="cuda") * torch.logspace(-3, 0, n, device="cuda")).to(dtype)
        _cuda.adamw8bit(pk, g, mq, vq, ms, vs, step, 1e-2, 0.9, 0.95, 1e-8, 0.1, scale)
        # the statement continues from the kernel's state, so that one differing code cannot compound over the steps
        ref.adamw8bit_step(pr, g.float(), mqr, vqr, msr, vsr, step, 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.5)
        assert (mq.int() - mqr.int()).abs().max() <= 1 and (vq.int() - vqr.int()).abs().max() <= 1
        assert ((mq != mqr).float().mean() < 0.01) and ((vq != vqr).float().mean() < 0.01)
        torch.testing.assert_close(ms, msr, rtol=1e-5, atol=0)
        torch.testing.assert_close(vs, vsr, rtol=1e-5, atol=0)
        torch.testing.assert_close(pk.float(), pr.to(dtype).float(), rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6)
        mqr.copy_(mq), vqr.copy_(vq), msr.copy_(ms), vsr.copy_(vs), pr.copy_(pk.float())
    m, v = ref.adamw8bit_decode(mq, vq, ms, vs, n)
    assert torch.isfinite(m).all() and torch.isfinite(v).all() and (v >= 0).all() and float(m.abs().max()) > 0


def test_adamw8bit_optimizer_trains_a_bf16_layer():
    from torchtune_b200.optim import AdamW8bit

    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    w_true = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16) * 0.2
    y = x @ w_true
    results = {}
    for name, cls in (("fp", torch.optim.AdamW), ("q", AdamW8bit)):
        torch.manual_seed(1)
        w = torch.nn.Parameter(torch.zeros(256, 128, device="cuda", dtype=torch.bfloat16))
        opt = cls([w], lr=3e-3, weight_decay=0.0)
        for _ in range(300):
            loss = ((x @ w - y).float() ** 2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
        results[name] = (loss.item(), opt)
    assert results["q"][0] < 1.5 * results["fp"][0] + 1e-3, (results["q"][0], results["fp"][0])
    assert results["q"][1].state_bytes() == 256 * 128 * 2 + 128 * 8


@pytest.mark.parametrize("cap,scale", [(0.0, 0.05), (3.0, 0.4)])
def test_token_logprobs(cap, scale):
    """``cap > 0``: log-softmax over cap·tanh(logits/cap) (Gemma-2), with weights large enough to put logits on the curved part."""
    T, D, V = 200, 256, 2048
    h = _rand(T, D, seed=1).requires_grad_()
    w = _rand(V, D, seed=2, scale=scale)
    labels = torch.randint(0, V, (4, 50), device="cuda")
    labels[:, :10] = -100
    lp = ops.token_logprobs(h.view(4, 50, D), w, labels, -100, 4, softcap=cap)
    g = _rand(4, 50, seed=3, dtype=torch.float32)
    (lp * g).sum().backward()
    hr = h.detach().float().requires_grad_()
    lpr = ref.token_logprobs(hr.view(4, 50, D), w.float(), labels, -100, 4, softcap=cap)
    (lpr * g).sum().backward()
    if cap:
        plain = ref.token_logprobs(hr.detach().view(4, 50, D), w.float(), labels, -100, 4)
        assert (plain - lpr.detach()).abs().max() > 0.5  # the cap changes these values, so the comparison below means something
    _close(lp, lpr, 1e-2, 2e-2, "logprobs")
    _close(h.grad, hr.grad, 5e-2, 5e-3, "logprobs dh")


# ------------------------------------------------------------------ optimizer
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_adamw_matches_torch(dtype):
    from torchtune_b200.optim import AdamW

    shapes = [(1000,), (256, 512), (7,), (4097, 3)]
    ps = [_rand(*s, seed=i, dtype=dtype) for i, s in enumerate(shapes)]
    mine = [p.clone().requires_grad_() for p in ps]
    theirs = [p.clone().requires_grad_() for p in ps]
    o1 = AdamW(mine, lr=1e-2, weight_decay=0.1)
    o2 = torch.optim.AdamW(theirs, lr=1e-2, weight_decay=0.1)
    for step in range(3):
        for i, (a, b) in enumerate(zip(mine, theirs)):
            g = _rand(*a.shape, seed=100 + 10 * step + i, dtype=dtype)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for a, b in zip(mine, theirs):
        _close(a, b, tol, tol, "adamw")


# ------------------------------------------------------------------ attention
def _attn_case(b, s, hq, hkv, d, mask, seed=0):
    q = _rand(b, s, hq, d, seed=seed).requires_grad_()
    k = _rand(b, s, hkv, d, seed=seed + 1).requires_grad_()
    v = _rand(b, s, hkv, d, seed=seed + 2).requires_grad_()
    go = _rand(b, s, hq, d, seed=seed + 3)
    o = ops.attention(q, k, v, mask)
    o.backward(go)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.attention(qr, kr, vr, causal=mask.causal, doc_ids=mask.doc_ids, chunk=mask.chunk, window=mask.window)
    orf.backward(go.float())
    _close(o, orf, 2e-2, 2e-2, "attn out")
    _close(v.grad, vr.grad, 3e-2, 3e-2, "attn dv")
    _close(k.grad, kr.grad, 3e-2, 5e-2, "attn dk")
    _close(q.grad, qr.grad, 3e-2, 5e-2, "attn dq")


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("s", [128, 384, 200])
def test_attention_causal(s, d):
    _attn_case(2, s, 4, 2, d, AttentionMask(causal=True))


def test_attention_noncausal():
    _attn_case(1, 256, 2, 2, 128, AttentionMask(causal=False))


def test_attention_packed_documents():
    mask = AttentionMask.from_seq_lens([[100, 156, 256], [512]]).to("cuda")
    _attn_case(2, 512, 8, 2, 128, mask)


def test_attention_chunk_and_window():
    _attn_case(1, 512, 4, 4, 64, AttentionMask(causal=True, chunk=192))
    _attn_case(1, 512, 4, 1, 128, AttentionMask(causal=True, window=100))


def test_attention_long():
    _attn_case(1, 2048, 8, 2, 128, AttentionMask(causal=True), seed=5)


# ------------------------------------------------------------------ model level
def test_tiny_llama_bf16_matches_fp32_reference():
    from helpers import TINY, fixed_init_
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss

    torch.manual_seed(0)
    model = llama3_1(**TINY)
    fixed_init_(model)
    tokens = torch.randint(0, 1024, (2, 128))
    labels = torch.randint(0, 1024, (2, 128))
    labels[:, :16] = -100

    def run(m, dev, use_ref):
        m = m.to(dev)
        loss_fn = LinearCrossEntropyLoss()
        loss_fn.set_model_output(m)
        ctx = ops.use_reference_ops() if use_ref else torch.enable_grad()
        with ctx:
            loss = loss_fn(m(tokens.to(dev)), labels.to(dev))
            loss.backward()
        m.skip_output_layer = False
        return loss.item(), {n: p.grad.float().cpu() for n, p in m.named_parameters()}

    import copy

    l_ref, g_ref = run(copy.deepcopy(model), "cpu", True)
    l_gpu, g_gpu = run(copy.deepcopy(model).to(torch.bfloat16), "cuda", False)
    assert abs(l_ref - l_gpu) < 5e-2, (l_ref, l_gpu)
    for n in g_ref:
        denom = g_ref[n].norm().item() + 1e-6
        rel = (g_ref[n] - g_gpu[n]).norm().item() / denom
        assert rel < 0.08, f"{n}: relative grad error {rel:.3f}"


# ------------------------------------------------------------------ data-parallel fused step
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_dp_reduce_adamw_bcast_emulated_ranks(world):
    """All ranks' buffers live on one GPU; the kernel is launched once per emulated rank (the
    launches do not wait on each other, so running them back to back is equivalent)."""
    import ctypes

    from torchtune_b200.ops._lib import check, lib, stream_ptr
    from torchtune_b200.parallel.dp import _declare_dp

    L = lib()
    _declare_dp(L)
    shard = 4096
    total = shard * world
    g = torch.Generator(device="cuda").manual_seed(world)
    p0 = (torch.randn(total, generator=g, device="cuda") * 0.1).bfloat16()
    params = [p0.clone() for _ in range(world)]
    grads = [(torch.randn(total, generator=g, device="cuda")).bfloat16() for _ in range(world)]
    m = [torch.zeros(shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    v = [torch.zeros(shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in grads])
    pp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in params])
    lr, b1, b2, eps, wd, scale = 1e-2, 0.9, 0.999, 1e-8, 0.1, 0.25
    for r in range(world):
        check(L.ttb_dp_reduce_adamw_bcast(gp, pp, world, r, r * shard, shard, m[r].data_ptr(), v[r].data_ptr(), None, None, None, scale, lr, b1, b2, eps, wd, 1.0 / (1 - b1), 1.0 / math.sqrt(1 - b2), 0, None, 0, 0, None, 0, 1, 0, stream_ptr()), "dp kernel")
    torch.cuda.synchronize()
    gsum = torch.stack([t.float() for t in grads]).sum(0) * scale
    want = p0.float().clone()
    mm, vv = torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
    ref.adamw_step(want, gsum, mm, vv, 1, lr, b1, b2, eps, wd)
    for r in range(world):
        _close(params[r], want, 1e-2, 1e-3, f"params on rank {r}")
    _close(torch.cat(m), mm, 2e-2, 1e-3, "exp_avg")

    # clipped variant: reduce -> norm -> update
    params2 = [p0.clone() for _ in range(world)]
    pp2 = (ctypes.c_void_p * world)(*[t.data_ptr() for t in params2])
    m2 = [torch.zeros(shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    v2 = [torch.zeros(shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    gs = [torch.empty(shard, dtype=torch.float32, device="cuda") for _ in range(world)]
    parts = [torch.empty(L.ttb_dp_grid(), dtype=torch.float32, device="cuda") for _ in range(world)]
    for r in range(world):
        check(L.ttb_dp_reduce_adamw_bcast(gp, pp2, world, r, r * shard, shard, m2[r].data_ptr(), v2[r].data_ptr(), gs[r].data_ptr(), parts[r].data_ptr(), None, 1.0, lr, b1, b2, eps, wd, 1.0, 1.0, 1, None, 0, 0, None, 0, 1, 0, stream_ptr()), "dp reduce")
    norm = torch.stack([p.sum() for p in parts]).sum().sqrt() * scale
    _close(norm, gsum.norm(), 1e-3, 1e-3, "global norm")
    coef = (torch.clamp(1.0 / (norm + 1e-6), max=1.0) * scale).reshape(1).float()
    for r in range(world):
        check(L.ttb_dp_reduce_adamw_bcast(gp, pp2, world, r, r * shard, shard, m2[r].data_ptr(), v2[r].data_ptr(), gs[r].data_ptr(), None, coef.data_ptr(), 1.0, lr, b1, b2, eps, wd, 1.0 / (1 - b1), 1.0 / math.sqrt(1 - b2), 2, None, 0, 0, None, 7, 1, 0, stream_ptr()), "dp update")
    want2 = p0.float().clone()
    mm, vv = torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
    ref.adamw_step(want2, gsum * float(torch.clamp(1.0 / (gsum.norm() + 1e-6), max=1.0)), mm, vv, 1, lr, b1, b2, eps, wd)
    for r in range(world):
        _close(params2[r], want2, 1e-2, 1e-3, f"clipped params on rank {r}")


@pytest.mark.parametrize("side_stream", [False, True])
def test_flat_engine_with_checkpointing_matches_plain_training(side_stream):
    """Flat store + direct weight-gradient delivery (+ side stream) + activation checkpointing
    give the same parameters after two steps as ordinary autograd with the multi-tensor AdamW."""
    import copy

    from helpers import TINY, fixed_init_
    from torchtune_b200 import training
    from torchtune_b200.engine.train_step import TrainStep
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules import TransformerSelfAttentionLayer
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss
    from torchtune_b200.ops import _cuda
    from torchtune_b200.optim import AdamW
    from torchtune_b200.parallel import DataParallelEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    base = llama3_1(**TINY)
    fixed_init_(base)
    base = base.to(torch.bfloat16).to(dev)
    tokens = torch.randint(0, 1024, (2, 128), device=dev)
    labels = torch.roll(tokens, -1, 1)
    batch = {"tokens": tokens, "labels": labels}

    plain = copy.deepcopy(base)
    lf1 = LinearCrossEntropyLoss()
    lf1.set_model_output(plain)
    s1 = TrainStep(plain, lf1, AdamW(plain.parameters(), lr=1e-3), dev)

    flat_model = copy.deepcopy(base)
    training.set_activation_checkpointing(flat_model, {TransformerSelfAttentionLayer})
    lf2 = LinearCrossEntropyLoss()
    lf2.set_model_output(flat_model)
    eng = DataParallelEngine(dev)
    eng.prepare(flat_model)
    _cuda.enable_direct_wgrad(True, use_side_stream=side_stream)
    s2 = TrainStep(flat_model, lf2, eng.build_optimizer(flat_model, lr=1e-3), dev, parallel=eng)
    try:
        for _ in range(2):
            l1 = s1.compute(dict(batch))
            l2 = s2.compute(dict(batch))
            assert abs(l1.item() - l2.item()) < 2e-2
        torch.cuda.synchronize()
        for (n, a), (_, b) in zip(plain.named_parameters(), flat_model.named_parameters()):
            _close(b, a, 2e-2, 3e-3, n)
    finally:
        _cuda.enable_direct_wgrad(False)
        del s2, flat_model
        eng.shutdown()


# ------------------------------------------------------------------ tensor-parallel GEMMs (ranks emulated on one GPU)
def _tp_lib():
    import ctypes

    from torchtune_b200.ops._lib import err_word, lib, stream_ptr
    from torchtune_b200.parallel.tp import _declare

    L = lib()
    _declare(L)
    return L, ctypes, err_word, stream_ptr


@pytest.mark.parametrize("world,rows,K,N", [(1, 256, 320, 192), (2, 256, 320, 192), (4, 256, 320, 192), (8, 256, 320, 192), (2, 1024, 512, 4096), (4, 512, 256, 2560)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_all_gather_fused_emulated_ranks(world, rows, K, N, b_mn):
    """Every emulated rank runs the all-gather → GEMM kernel over the same set of shard buffers (here all on one
    device; on a real group they are peer mappings).  Launches are sequential and never wait on each other.  The two
    large shapes give every persistent CTA several tiles (accumulator double-buffering and the piece counters at work)."""
    from torchtune_b200.ops._lib import check_device_errors

    L, ctypes, err_word, stream_ptr = _tp_lib()
    shards = [_rand(rows, K, scale=0.5, seed=10 + r) for r in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in shards])
    full = torch.cat(shards).float()
    for rank in range(world):
        w = _rand(K, N, scale=0.1, seed=50 + rank) if b_mn else _rand(N, K, scale=0.1, seed=50 + rank)
        bias = _rand(N, scale=0.1, seed=70 + rank)
        out = torch.empty(world * rows, N, dtype=torch.bfloat16, device="cuda")
        gathered = torch.full((world * rows, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        sync = torch.full((1 + world * rows // 128,), 7, dtype=torch.int32, device="cuda")  # the entry point zeroes it
        gather_own = rank % 2
        rc = L.ttb_gemm_ag_bf16(ptrs, w.data_ptr(), out.data_ptr(), gathered.data_ptr(), sync.data_ptr(), gather_own, world, rank, rows, N, K, int(b_mn),
                                w.stride(0), N, bias.data_ptr(), None, 0, 0, 0, err_word(out.device).data_ptr(), stream_ptr())
        assert rc == 0
        want = (full @ w.float() if b_mn else full @ w.float().t()) + bias.float()
        _close(out, want, 2e-2, 2e-2, f"ag_gemm rank {rank}")
        # the gathered activation is a by-product: remote rows always, own rows on request
        own = slice(rank * rows, (rank + 1) * rows)
        mask = torch.ones(world * rows, dtype=torch.bool, device="cuda")
        if not gather_own:
            mask[own] = False
            assert torch.isnan(gathered[own].float()).all()
        assert torch.equal(gathered[mask].float(), full[mask])
    check_device_errors()


@pytest.mark.parametrize("world,rows,K,N", [(1, 128, 192, 256), (2, 128, 192, 256), (4, 128, 192, 256), (8, 128, 192, 256), (2, 1024, 256, 3072), (4, 256, 320, 200)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_reduce_scatter_fused_emulated_ranks(world, rows, K, N, b_mn):
    """The large shape gives every persistent CTA several tiles (staging buffers of the TMA-store epilogue are reused); N = 200
    ends inside a 64-column store box (clipped by the tensor map)."""
    L, ctypes, err_word, stream_ptr = _tp_lib()
    T = world * rows
    staging = [torch.full((world, rows, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in staging])
    xs = [_rand(T, K, scale=0.5, seed=20 + r) for r in range(world)]
    ws = [(_rand(K, N, scale=0.1, seed=40 + r) if b_mn else _rand(N, K, scale=0.1, seed=40 + r)) for r in range(world)]
    for rank in range(world):
        rc = L.ttb_gemm_rs_bf16(xs[rank].data_ptr(), ws[rank].data_ptr(), ptrs, world, rank, rows, N, K, int(b_mn), K, ws[rank].stride(0), N, err_word(xs[0].device).data_ptr(), stream_ptr())
        assert rc == 0
    total = sum((x.float() @ w.float()) if b_mn else (x.float() @ w.float().t()) for x, w in zip(xs, ws))
    for owner in range(world):
        residual = _rand(rows, N, scale=0.3, seed=90 + owner)
        bias = _rand(N, scale=0.1, seed=95 + owner)
        out = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
        rc = L.ttb_rs_reduce(staging[owner].data_ptr(), residual.data_ptr(), bias.data_ptr(), out.data_ptr(), world, rows, N, N, N, N, None, 0, 0, 0, owner, None, stream_ptr())
        assert rc == 0
        want = total[owner * rows : (owner + 1) * rows] + residual.float() + bias.float()
        _close(out, want, 3e-2, 3e-2 * max(1, world // 2), f"gemm_rs owner {owner}")


def test_tp_context_single_rank_matches_plain_linear():
    """World size 1 exercises the whole fused path (peer buffers, barrier no-op, kernels) against ``F.linear``."""
    from torchtune_b200.parallel.tp import TensorParallelContext, column_parallel_linear, row_parallel_linear

    tp = TensorParallelContext(torch.device("cuda", torch.cuda.current_device()), max_rows_per_rank=256, max_width=512)
    try:
        x = _rand(256, 384, scale=0.5, seed=1).requires_grad_()
        w1 = _rand(512, 384, scale=0.1, seed=2).requires_grad_()
        w2 = _rand(384, 512, scale=0.1, seed=3).requires_grad_()
        h = column_parallel_linear(x, w1, tp)
        y = row_parallel_linear(h, w2, tp, residual=x)
        y.float().sum().backward()
        xf, w1f, w2f = (t.detach().float().requires_grad_() for t in (x, w1, w2))
        yf = (xf @ w1f.t()).bfloat16().float() @ w2f.t() + xf
        yf.sum().backward()
        _close(y, yf, 3e-2, 3e-2, "tp forward")
        _close(x.grad, xf.grad, 5e-2, 5e-2, "tp dx")
        _close(w1.grad, w1f.grad, 5e-2, 2e-1, "tp dw1")
    finally:
        tp.close()


# ----------------------------------------------------------------------------- MoE index kernels, embedding
@pytest.mark.parametrize("n,E", [(1, 4), (700, 16), (5000, 128), (8192, 8)])
def test_moe_route_sort_matches_stable_argsort(n, E):
    from torchtune_b200.ops._cuda import moe_route_sort

    g = torch.Generator(device="cuda").manual_seed(n)
    ids = torch.randint(0, E, (n,), generator=g, device="cuda")
    counts, order = moe_route_sort(ids, E)
    assert torch.equal(counts, torch.bincount(ids, minlength=E))
    assert torch.equal(order, torch.argsort(ids, stable=True))


@pytest.mark.parametrize("R,E,align", [(1, 4, 16), (8, 2, 16), (4, 16, 128), (2, 3, 8)])
def test_moe_permute_indices_matches_loop_oracle(R, E, align):
    from torchtune_b200.modules.moe.indices import fill_indices_cpu, generate_permute_indices

    g = torch.Generator().manual_seed(R * 100 + E)
    counts = torch.randint(0, 40, (R * E,), generator=g)
    counts[0] = 0
    max_len = int(counts.sum()) + E * align
    got, sizes, offs = generate_permute_indices(counts.cuda(), E, R, max_len, align)
    want, wsizes, woffs = generate_permute_indices(counts, E, R, max_len, align, use_cpu=True)
    assert torch.equal(got.cpu(), want) and torch.equal(sizes.cpu(), wsizes) and torch.equal(offs.cpu(), woffs)
    start = (counts.cumsum(0) - counts)
    loop = fill_indices_cpu(counts, start, woffs - wsizes, E, R, max_len)
    assert torch.equal(got.cpu(), loop)


def test_embedding_matches_reference_with_repeated_tokens():
    g = torch.Generator(device="cuda").manual_seed(3)
    V, D = 1000, 4096 + 64
    table = (torch.randn(V, D, generator=g, device="cuda") * 0.1).bfloat16().requires_grad_()
    ids = torch.randint(0, V, (4, 333), generator=g, device="cuda")
    ids[:, :50] = 7  # a frequent token: 200 rows summed into one table row
    out = ops.embedding(ids, table)
    dy = (torch.randn(4, 333, D, generator=g, device="cuda") * 0.1).bfloat16()
    out.backward(dy)
    tf = table.detach().float().requires_grad_()
    ref = torch.nn.functional.embedding(ids, tf)
    ref.backward(dy.float())
    assert torch.equal(out.float(), ref)
    rel = (table.grad.float() - tf.grad).norm() / tf.grad.norm()
    assert rel < 4e-3


# ----------------------------------------------------------------------------- expert-parallel exchange (ranks emulated on one GPU)
@pytest.mark.parametrize("world,E,k", [(1, 4, 1), (2, 4, 2), (4, 16, 1), (8, 16, 2)])
def test_expert_parallel_plan_push_pull_emulated_ranks(world, E, k):
    import ctypes

    from torchtune_b200.ops._lib import lib, stream_ptr
    from torchtune_b200.parallel.ep import _declare

    L = lib()
    _declare(L)
    T, dim = 96, 264
    pairs = T * k
    cap = world * pairs
    g = torch.Generator(device="cuda").manual_seed(world * 10 + k)
    xs = [_rand(T, dim, scale=0.5, seed=300 + r) for r in range(world)]
    experts, tokens, scales, counts = [], [], [], []
    for r in range(world):
        e = torch.randint(0, E, (pairs,), generator=g, device="cuda")
        if r == 0:
            e[e == 1] = 0  # an expert that receives nothing from rank 0
        order = torch.argsort(e, stable=True)
        experts.append(e[order])
        tokens.append((order // k).contiguous())
        scales.append(_rand(pairs, scale=1.0, seed=400 + r))
        counts.append(torch.bincount(e, minlength=E))
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    recv = [torch.full((cap, dim), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    plans = []
    for r in range(world):
        dr = torch.empty(pairs, dtype=torch.int32, device="cuda")
        drow = torch.empty(pairs, dtype=torch.int32, device="cuda")
        rc_counts = torch.empty(E // world, dtype=torch.int64, device="cuda")
        rc_total = torch.empty(1, dtype=torch.int32, device="cuda")
        assert L.ttb_ep_plan(arr(counts), world, r, E, pairs, dr.data_ptr(), drow.data_ptr(), rc_counts.data_ptr(), rc_total.data_ptr(), stream_ptr()) == 0
        plans.append((dr, drow, rc_counts, rc_total))
        assert L.ttb_ep_push(xs[r].data_ptr(), tokens[r].data_ptr(), scales[r].data_ptr(), dr.data_ptr(), drow.data_ptr(), arr(recv), world, pairs, dim, cap, stream_ptr()) == 0
    epr = E // world
    all_counts = torch.stack(counts)  # [world, E]
    for d in range(world):
        want_rows = []
        for e in range(d * epr, (d + 1) * epr):
            for r in range(world):
                sel = experts[r] == e
                want_rows.append((xs[r][tokens[r][sel]].float() * scales[r][sel].float()[:, None]).bfloat16())
        want = torch.cat(want_rows)
        assert torch.equal(plans[d][2], all_counts[:, d * epr : (d + 1) * epr].sum(0))
        assert int(plans[d][3]) == want.shape[0]
        assert torch.equal(recv[d][: want.shape[0]], want)
        assert torch.isnan(recv[d][want.shape[0] :].float()).all()
    result = [(t.float() * 2).bfloat16() for t in recv]
    for r in range(world):
        out = torch.empty(pairs, dim, dtype=torch.bfloat16, device="cuda")
        assert L.ttb_ep_pull(arr(result), world, plans[r][0].data_ptr(), plans[r][1].data_ptr(), out.data_ptr(), pairs, dim, cap, stream_ptr()) == 0
        want = ((xs[r][tokens[r]].float() * scales[r].float()[:, None]).bfloat16().float() * 2).bfloat16()
        assert torch.equal(out, want)


# ----------------------------------------------------------------------------- fp8 GEMM + cast/transpose
def _fp8_ref(t, scale, dtype):
    return (t.float() * scale).clamp(-torch.finfo(dtype).max, torch.finfo(dtype).max).to(dtype)


@pytest.mark.parametrize("e5m2", [False, True])
@pytest.mark.parametrize("rowwise", [False, True])
def test_fp8_cast_transpose_matches_torch(e5m2, rowwise):
    from torchtune_b200.ops._cuda import fp8_cast, fp8_scales

    dtype = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    x = _rand(208, 336, scale=2.0, seed=5)
    s_row, s_col = fp8_scales(x, e5m2, rowwise)
    out, out_t = fp8_cast(x, s_row, s_col, e5m2=e5m2)
    want = _fp8_ref(x, s_row.reshape(-1, 1) if rowwise else s_row, dtype)
    want_t = _fp8_ref(x, s_col.reshape(1, -1) if rowwise else s_col, dtype).t().contiguous()
    assert torch.equal(out.view(dtype).float(), want.float())
    assert torch.equal(out_t.view(dtype).float(), want_t.float())


@pytest.mark.parametrize("M,N,K", [(128, 64, 128), (384, 272, 208), (1024, 1024, 2048), (2048, 4096, 512)])
@pytest.mark.parametrize("rowwise", [False, True])
def test_gemm_fp8_matches_dequantised_fp32(M, N, K, rowwise):
    """The kernel must reproduce the product of the *quantised* operands exactly up to fp32 accumulation order."""
    from torchtune_b200.ops._cuda import fp8_cast, fp8_scales, gemm_fp8
    from torchtune_b200.ops._lib import check_device_errors

    a, b = _rand(M, K, scale=1.0, seed=1), _rand(N, K, scale=0.5, seed=2)
    bias = _rand(N, scale=0.5, seed=3)
    sa, _ = fp8_scales(a, False, rowwise)
    sb, _ = fp8_scales(b, True, rowwise)
    aq, _ = fp8_cast(a, sa, sa, want_t=False)
    bq, _ = fp8_cast(b, sb, sb, e5m2=True, want_t=False)
    got = gemm_fp8(aq, bq, 1.0 / sa, 1.0 / sb, b_e5m2=True, bias=bias)
    check_device_errors()
    af = aq.view(torch.float8_e4m3fn).float() / (sa.reshape(-1, 1) if rowwise else sa)
    bf = bq.view(torch.float8_e5m2).float() / (sb.reshape(-1, 1) if rowwise else sb)
    want = af @ bf.t() + bias.float()
    _close(got, want, 1e-2, 1e-2 * want.abs().max().item(), "gemm_fp8")


@pytest.mark.parametrize("rowwise", [False, True])
def test_fp8_linear_forward_backward_close_to_bf16(rowwise):
    x = _rand(4, 128, 512, scale=1.0, seed=7).requires_grad_()
    w = _rand(768, 512, scale=0.05, seed=8).requires_grad_()
    bias = _rand(768, scale=0.1, seed=9).requires_grad_()
    y = ops.fp8_linear(x, w, bias, rowwise=rowwise)
    assert y is not None and y.shape == (4, 128, 768)
    dy = _rand(4, 128, 768, scale=0.1, seed=10)
    y.backward(dy)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yf = torch.nn.functional.linear(xf, wf, bf)
    yf.backward(dy.float())
    rel = lambda a, b: float((a.float() - b).norm() / b.norm())
    assert rel(y, yf) < 0.06 and rel(x.grad, xf.grad) < 0.12 and rel(w.grad, wf.grad) < 0.12, (rel(y, yf), rel(x.grad, xf.grad), rel(w.grad, wf.grad))
    assert rel(bias.grad, bf.grad) < 1e-2


# ----------------------------------------------------------------------------- failure detection: a bounded device wait that runs out
def test_dp_bucket_wait_times_out_with_error_status_and_leaves_state_untouched():
    """A peer that never declares its bucket final: the wait in front of the bucket kernel gives up after its cycle budget and stores
    an error code, every CTA of the bucket kernel sees it and returns, the host turns the code into an exception, and neither
    parameters nor optimizer state are modified.  The context stays usable."""
    import ctypes

    from torchtune_b200.ops._lib import KernelError, check, check_device_errors, err_word, lib, stream_ptr
    from torchtune_b200.parallel.dp import _declare_dp

    L = lib()
    _declare_dp(L)
    world, n = 2, 4096
    grads = [_rand(n, seed=r) for r in range(world)]
    params = [_rand(n, seed=10) for _ in range(world)]
    before = params[0].clone()
    m, v = torch.zeros(n // 2, dtype=torch.bfloat16, device="cuda"), torch.zeros(n // 2, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(world * L.ttb_dp_max_buckets(), dtype=torch.int32, device="cuda")  # nobody ever writes epoch 1 here
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    pp = (ctypes.c_void_p * world)(*[p.data_ptr() for p in params])
    L.ttb_dp_set_wait_cycles(200_000_000)  # ≈ 0.1 s
    try:
        check(L.ttb_dp_reduce_adamw_bcast(gp, pp, world, 0, 0, n // 2, m.data_ptr(), v.data_ptr(), None, None, None, 1.0, 1e-3, 0.9, 0.999, 1e-8, 0.01, 10.0, 31.6, 0,
                                          flags.data_ptr(), 3, 1, err_word(flags.device).data_ptr(), 0, 1, 0, stream_ptr()), "dp kernel")
        with pytest.raises(KernelError, match="201"):
            check_device_errors()
    finally:
        L.ttb_dp_set_wait_cycles(0)  # back to the default budget
    assert torch.equal(params[0], before) and not m.any() and not v.any()
    check_device_errors()  # the error word was cleared; the device keeps working
    assert torch.isfinite(_rand(8, 8).float() @ _rand(8, 8).float()).all()


# ----------------------------------------------------------------------------- weight all-gather → GEMM (ranks emulated on one GPU)
@pytest.mark.parametrize("world,rows,K,M", [(1, 256, 320, 200), (2, 256, 320, 384), (4, 256, 192, 128), (8, 256, 256, 2304), (2, 1792, 512, 1024), (1, 64, 128, 256), (1, 128, 128, 256)])
def test_gemm_weight_gather_fused_emulated_ranks(world, rows, K, M):
    """Every emulated rank multiplies its own activations with the weight whose row shards live in `world` buffers (peer mappings
    on a real group): remote shards are pulled by the kernel's copier warps, the own shard is read in place."""
    import ctypes

    from torchtune_b200.ops._lib import check_device_errors, err_word, lib, stream_ptr
    from torchtune_b200.parallel.fsdp import _declare

    L = lib()
    _declare(L)
    N = world * rows
    shards = [_rand(rows, K, scale=0.1, seed=30 + r) for r in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in shards])
    w_full = torch.cat(shards).float()
    for rank in range(world):
        x = _rand(M, K, scale=0.5, seed=60 + rank)
        bias = _rand(N, scale=0.1, seed=80 + rank)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        gathered = torch.full((N, K), float("nan"), dtype=torch.bfloat16, device="cuda")
        sync = torch.full((2 + N // 64,), 5, dtype=torch.int32, device="cuda")
        rc = L.ttb_gemm_wg_bf16(x.data_ptr(), ptrs, out.data_ptr(), gathered.data_ptr(), sync.data_ptr(), world, rank, rows, M, K, K, N, bias.data_ptr(),
                                err_word(out.device).data_ptr(), stream_ptr())
        assert rc == 0
        _close(out, x.float() @ w_full.t() + bias.float(), 2e-2, 2e-2, f"wg_gemm rank {rank}")
        remote = torch.ones(N, dtype=torch.bool, device="cuda")
        remote[rank * rows : (rank + 1) * rows] = False
        assert torch.equal(gathered[remote].float(), w_full[remote])
    check_device_errors()


# ----------------------------------------------------------------------------- two operand pairs, one accumulator (LoRA-fused GEMM)
@pytest.mark.parametrize("M,N,K,K2", [(256, 320, 192, 64), (1000, 512, 1024, 8), (2048, 4096, 512, 96),
                                      (8192, 4096, 1024, 64), (4100, 6152, 512, 24)])  # the last two are large enough for the CTA-pair kernel
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_dual_matches_sum_of_products(M, N, K, K2, b_mn):
    from torchtune_b200.ops._cuda import gemm_dual
    from torchtune_b200.ops._lib import check_device_errors

    a, a2 = _rand(M, K, scale=0.5, seed=1), _rand(M, K2, scale=0.5, seed=2)
    b = _rand(K, N, scale=0.1, seed=3) if b_mn else _rand(N, K, scale=0.1, seed=3)
    b2 = _rand(K2, N, scale=0.1, seed=4) if b_mn else _rand(N, K2, scale=0.1, seed=4)
    bias = _rand(N, scale=0.2, seed=5)
    got = gemm_dual(a, b, a2, b2, b_mn=b_mn, bias=bias)
    check_device_errors()
    want = (a.float() @ b.float() + a2.float() @ b2.float()) if b_mn else (a.float() @ b.float().t() + a2.float() @ b2.float().t())
    _close(got, want + bias.float(), 2e-2, 2e-2, "gemm_dual")


def test_nf4_quantize_kernels_match_reference():
    from torchtune_b200.ops._cuda import nf4_quantize

    w = _rand(256, 1024, scale=0.05, seed=3)
    w[0, :64] = 0  # an all-zero block
    got = nf4_quantize(w, 64, 256)
    want = ref.nf4_quantize(w, 64, 256)
    assert torch.equal(got[1], want[1]) and torch.allclose(got[2], want[2]) and torch.allclose(got[3], want[3])
    mismatch = (got[0] != want[0]).float().mean().item()
    assert mismatch < 1e-4, mismatch  # identical up to values that sit exactly on a midpoint after fp32 rounding
    back = ref.nf4_dequantize(got[0], got[1], got[2], got[3], w.shape, 64, 256, torch.float32)
    assert (back - w.float()).abs().max() < 0.2 * w.float().abs().max()


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(64, 4096, 8192, True, True), (4096, 64, 8192, True, True), (128, 256, 4096 + 64, False, False), (200, 72, 1000, False, True)])
def test_gemm_split_k_matches_fp32(M, N, K, a_mn, b_mn):
    from torchtune_b200.ops._cuda import gemm_skinny
    from torchtune_b200.ops._lib import check_device_errors

    a = _rand(K, M, scale=0.3, seed=1) if a_mn else _rand(M, K, scale=0.3, seed=1)
    b = _rand(K, N, scale=0.3, seed=2) if b_mn else _rand(N, K, scale=0.3, seed=2)
    got = gemm_skinny(a, b, a_mn=a_mn, b_mn=b_mn, alpha=0.5)
    check_device_errors()
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    _close(got, 0.5 * (af @ bf), 2e-2, 2e-2 * (K ** 0.5) * 0.1, "split-k")


def test_peer_buffer_guard_regions_detect_writes_outside(monkeypatch):
    """Debug aid for the peer-memory kernels: with TTB_PEER_GUARD_BYTES set, every peer buffer sits between two pattern-filled
    regions of the same allocation; a data-parallel step must leave them intact, and a stray write next to the buffer is reported."""
    from torchtune_b200.ops._lib import KernelError
    from torchtune_b200.parallel.dp import DataParallelEngine
    from torchtune_b200.parallel.fabric import PeerBuffer

    monkeypatch.setenv("TTB_PEER_GUARD_BYTES", "1000")
    dev = torch.device("cuda", 0)
    buf = PeerBuffer(4096 + 24, dev)
    assert buf.guard == 1024 and buf.local_ptr % 256 == 0
    buf.tensor(torch.uint8).fill_(7)  # the whole usable range
    buf.check_guards()
    buf._whole[buf.guard + buf.nbytes + 5] = 1  # inside the allocation, outside the buffer
    with pytest.raises(KernelError, match="above were overwritten"):
        buf.check_guards()
    with pytest.raises(KernelError):
        buf.close()
    assert buf.local_ptr == 0  # freed all the same

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.Linear(512, 256)).to(dev).bfloat16()
    engine = DataParallelEngine(device=dev, group=None)
    engine.prepare(model)
    opt = engine.build_optimizer(model, lr=1e-3)
    for _ in range(2):
        model(torch.randn(64, 256, device=dev, dtype=torch.bfloat16)).float().pow(2).mean().backward()
        engine.optimizer_step(model, opt, 1.0, 1.0)
    engine.flat.param_buf.check_guards()
    engine.flat.grad_buf.check_guards()
    engine.shutdown()


def _attn_general(b, s, sk, hq, hkv, d, mask, softcap=0.0, seed=0, grads=True):
    """Native attention against the fp32 PyTorch statement for query length ≠ key length, boolean masks and soft-capping."""
    q = _rand(b, s, hq, d, seed=seed).requires_grad_(grads)
    k = _rand(b, sk, hkv, d, seed=seed + 1).requires_grad_(grads)
    v = _rand(b, sk, hkv, d, seed=seed + 2).requires_grad_(grads)
    before = dict(ops.fallback_counts)
    o = ops.attention(q, k, v, mask, softcap=softcap)
    assert dict(ops.fallback_counts) == before, "the call left the sm_100a kernels"
    qr, kr, vr = (t.detach().float().requires_grad_(grads) for t in (q, k, v))
    orf = ref.attention(qr, kr, vr, causal=mask.causal, doc_ids=mask.doc_ids, chunk=mask.chunk, window=mask.window, bool_mask=mask.bool_mask, softcap=softcap)
    _close(o, orf, 2e-2, 2e-2, "attn out")
    if grads:
        go = _rand(b, s, hq, d, seed=seed + 3)
        o.backward(go)
        orf.backward(go.float())
        _close(v.grad, vr.grad, 3e-2, 3e-2, "attn dv")
        _close(k.grad, kr.grad, 3e-2, 5e-2, "attn dk")
        _close(q.grad, qr.grad, 3e-2, 5e-2, "attn dq")


def test_attention_benchmark_shape_packed_512_token_documents():
    """The headline benchmark's own attention call: 4 × 2048 tokens, 32 / 8 heads, documents of 512 tokens."""
    doc_ids = torch.arange(4, dtype=torch.int32, device="cuda").repeat_interleave(512).view(1, 2048).expand(4, 2048).contiguous()
    _attn_case(4, 2048, 32, 8, 128, AttentionMask(causal=True, doc_ids=doc_ids), seed=11)


@pytest.mark.parametrize("d", [128, 64])
def test_attention_cross_attention_unmasked_and_masked(d):
    """Query length ≠ key length (Llama-3.2-Vision cross-attention): no mask, then a boolean mask that hides whole key ranges
    per query (each text token sees the tiles of its own image only) including rows that see nothing."""
    _attn_general(2, 200, 333, 8, 2, d, AttentionMask(causal=False))
    g = torch.Generator().manual_seed(3)
    m = torch.zeros(2, 200, 333, dtype=torch.bool)
    for bi in range(2):
        for start in range(0, 200, 50):
            lo = int(torch.randint(0, 200, (1,), generator=g))
            m[bi, start : start + 50, lo : lo + 120] = True
    m[0, 7] = False  # a query without any visible key: output and gradients are zero
    _attn_general(2, 200, 333, 8, 2, d, AttentionMask(causal=False, bool_mask=m.cuda()), seed=4)


def test_attention_cached_decoding_steps():
    """One and a few new tokens against a partly filled KV cache: boolean ``[b, s_q, max_seq]`` masks as the decoder builds them
    (rows of the causal matrix picked by position), and the causal flag with fewer queries than keys."""
    max_seq, filled = 640, 301
    causal = torch.tril(torch.ones(max_seq, max_seq, dtype=torch.bool))
    for s_q in (1, 5):
        pos = torch.arange(filled - s_q, filled)
        m = causal[pos].unsqueeze(0).expand(3, s_q, max_seq).contiguous().cuda()
        _attn_general(3, s_q, max_seq, 8, 2, 128, AttentionMask(causal=False, bool_mask=m), seed=20 + s_q, grads=False)
    _attn_general(2, 5, 261, 4, 4, 64, AttentionMask(causal=True), seed=30)


def test_attention_arbitrary_boolean_mask_with_gradients():
    g = torch.Generator().manual_seed(5)
    m = torch.rand(2, 256, 256, generator=g) < 0.3
    m |= torch.eye(256, dtype=torch.bool)
    _attn_general(2, 256, 256, 4, 2, 128, AttentionMask(causal=False, bool_mask=m.cuda()), seed=40)


@pytest.mark.parametrize("mask", [AttentionMask(causal=True), AttentionMask(causal=True, window=100)])
def test_attention_softcap(mask):
    """Gemma-2 style soft-capped scores (tanh inside the softmax warps; its derivative in the backward pass)."""
    _attn_general(2, 384, 384, 4, 2, 128, mask, softcap=30.0, seed=50)
    _attn_general(1, 200, 200, 4, 4, 64, mask, softcap=5.0, seed=51)


# ------------------------------------------------------------------ gate / up projections with SwiGLU in the GEMM epilogue
@pytest.mark.parametrize("M,K,N", [(2048, 512, 4864), (4096, 1024, 2688), (2304, 328, 4104)])
def test_gate_up_swiglu_fused_gemm(M, K, N):
    """One CTA-pair GEMM whose two B halves are the gate and the up projection, SwiGLU in the epilogue: forward value with and
    without gradients, and the gradients of x, W1, W3 against fp32."""
    from torchtune_b200.ops._cuda import gate_up_swiglu

    x = _rand(M, K, seed=1, scale=0.5).requires_grad_()
    w1 = _rand(N, K, seed=2, scale=0.05).requires_grad_()
    w3 = _rand(N, K, seed=3, scale=0.05).requires_grad_()
    with torch.no_grad():
        h0 = gate_up_swiglu(x, w1, w3)
    assert h0 is not None, "shape was expected to qualify for the fused kernel"
    h = gate_up_swiglu(x, w1, w3)
    assert torch.equal(h, h0)  # the gradient-free pass (no pre-activations stored) computes the same values
    dh = _rand(M, N, seed=4, scale=0.1)
    h.backward(dh)
    xr, w1r, w3r = (t.detach().float().requires_grad_() for t in (x, w1, w3))
    g, u = xr @ w1r.t(), xr @ w3r.t()
    hr = torch.nn.functional.silu(g) * u
    hr.backward(dh.float())
    _close(h, hr, 3e-2, 3e-2, "fused swiglu fwd")
    _close(x.grad, xr.grad, 3e-2, 5e-2, "fused swiglu dx")
    _close(w1.grad, w1r.grad, 3e-2, 0.3, "fused swiglu dw1")
    _close(w3.grad, w3r.grad, 3e-2, 0.3, "fused swiglu dw3")


# ------------------------------------------------------------------ MoE routing and row kernels
@pytest.mark.parametrize("T,E,k", [(1000, 16, 1), (513, 8, 2), (64, 128, 4)])
def test_moe_route_kernel_matches_sigmoid_topk(T, E, k):
    from torchtune_b200.ops._cuda import moe_route

    logits = _rand(T, E, seed=1, scale=2.0).requires_grad_()
    scores, selected = moe_route(logits, k)
    ref_scores = torch.sigmoid(logits.detach().float()).to(torch.bfloat16)
    want_s, want_i = torch.topk(ref_scores, k=k, dim=1)
    assert torch.equal(scores, want_s)  # values are unique up to ties; tied experts may differ in index, never in score
    assert torch.equal(ref_scores.gather(1, selected), want_s)
    dscores = _rand(T, k, seed=2)
    scores.backward(dscores)
    lr = logits.detach().float().requires_grad_()
    torch.sigmoid(lr).gather(1, selected).backward(dscores.float())
    _close(logits.grad, lr.grad, 3e-2, 1e-3, "router logit gradient")


def test_moe_gather_and_combine_row_kernels():
    """Permute·score and un-permute + sum against index_select / index_add, forward and backward, top-2 routing."""
    from torchtune_b200.ops._cuda import moe_combine, moe_gather, moe_route_sort

    T, D, E, k = 300, 256, 8, 2
    x = _rand(T, D, seed=1).requires_grad_()
    sel = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
    scores = torch.rand(T, k, device="cuda").to(torch.bfloat16).requires_grad_()
    counts, order, inv = moe_route_sort(sel.reshape(-1), E, with_inverse=True)
    assert torch.equal(inv[order], torch.arange(T * k, device="cuda")) and counts.sum().item() == T * k
    token_idx = order // k
    top = scores.reshape(-1)[order]
    routed = moe_gather(x, token_idx, top, inv, k)
    base = _rand(T, D, seed=3).requires_grad_()
    w = _rand(T * k, D, seed=4, scale=0.5)
    out = moe_combine(routed * w, inv, token_idx, base, k)
    go = _rand(T, D, seed=5)
    out.backward(go)

    xr, sr, br = (t.detach().float().requires_grad_() for t in (x, scores, base))
    routed_r = xr.index_select(0, token_idx) * sr.reshape(-1)[order].reshape(-1, 1)
    out_r = br.index_add(0, token_idx, routed_r * w.float())
    out_r.backward(go.float())
    _close(routed, routed_r, 2e-2, 2e-2, "gather·score")
    _close(out, out_r, 3e-2, 5e-2, "combine")
    _close(x.grad, xr.grad, 3e-2, 5e-2, "dx")
    _close(base.grad, br.grad, 1e-2, 1e-2, "dbase")
    _close(scores.grad, sr.grad, 5e-2, 0.3, "dscores")


# ----------------------------------------------------------------------------- block-scaled (MX) fp8
@pytest.mark.parametrize("R,C,transpose", [(256, 512, False), (130, 96, False), (8, 4096, False), (256, 512, True), (160, 200, True), (4096, 24, True)])
def test_mx_quantize_matches_oracle(R, C, transpose):
    from torchtune_b200.ops._cuda import mx_quantize, mx_unpack_scales

    x = _rand(R, C, seed=3, scale=2.0)
    x[0, :] = 0  # all-zero blocks
    x[1, 5] = 300.0  # an outlier that only its own block pays for
    q, sf = mx_quantize(x, transpose=transpose)
    want_q, want_e = ref.mx_quantize(x, transpose=transpose)
    rows, k = want_q.shape
    assert q.shape == (rows, k)
    assert torch.equal(mx_unpack_scales(sf, rows, k), want_e)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), want_q)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 4096), (520, 264, 160), (8192, 4096, 1024), (96, 40, 32)])
def test_gemm_mxfp8_matches_dequantized_matmul(M, N, K):
    from torchtune_b200.ops._cuda import gemm_mxfp8, mx_quantize
    from torchtune_b200.ops._lib import check_device_errors

    a, b = _rand(M, K, seed=1, scale=1.5), _rand(N, K, seed=2, scale=0.1)
    a[:, : K // 2] *= 40.0  # very different magnitudes between blocks: a wrong scale id or row mapping shows up at once
    bias = _rand(N, seed=3, scale=0.5)
    aq, asf = mx_quantize(a)
    bq, bsf = mx_quantize(b)
    got = gemm_mxfp8(aq, asf, bq, bsf, bias=bias)
    check_device_errors()
    want = ref.mx_roundtrip(a) @ ref.mx_roundtrip(b).t() + bias.float()
    _close(got, want, 1e-2, 1e-2 * want.abs().max().item(), "gemm_mxfp8")
    again = gemm_mxfp8(aq, asf, bq, bsf, out=got.clone(), accumulate=True)
    _close(again, 2 * want - bias.float(), 2e-2, 2e-2 * want.abs().max().item(), "gemm_mxfp8 accumulate")


def test_mxfp8_linear_autograd_close_to_bf16():
    x = _rand(4, 64, 512, seed=8).requires_grad_()
    w = _rand(768, 512, seed=9, scale=0.05).requires_grad_()
    bias = _rand(768, seed=10).requires_grad_()
    y = ops.mxfp8_linear(x, w, bias)
    assert y is not None
    gy = _rand(4, 64, 768, seed=11)
    y.backward(gy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(gy.float())
    for name, got, want in (("y", y, yr), ("dx", x.grad, xr.grad), ("dw", w.grad, wr.grad), ("db", bias.grad, br.grad)):
        rel = (got.float() - want).norm() / want.norm()
        assert rel < 0.06, (name, rel.item())  # e4m3 has 3 mantissa bits: about 3 % relative error per operand


def test_mxfp8_linear_shares_the_quantised_activation_between_projections():
    from torchtune_b200.ops import _cuda

    x = _rand(256, 512, seed=21)
    w1, w2 = _rand(384, 512, seed=22, scale=0.05), _rand(640, 512, seed=23, scale=0.05)
    _cuda.mx_clear_shared()
    y1 = ops.mxfp8_linear(x, w1)
    hit = _cuda._MX_LAST[False][2]
    y2 = ops.mxfp8_linear(x, w2)  # same activation, other weight: served from the shared entry
    assert _cuda._MX_LAST[False][2] is hit
    _cuda.mx_clear_shared()
    assert torch.equal(y2, ops.mxfp8_linear(x, w2)) and torch.equal(y1, ops.mxfp8_linear(x, w1))
    x.add_(1.0)  # an in-place change must not be served from the entry
    y3 = ops.mxfp8_linear(x, w2)
    _cuda.mx_clear_shared()
    assert torch.equal(y3, ops.mxfp8_linear(x, w2))


@pytest.mark.parametrize("R,C", [(256, 512), (96, 32), (8192, 1024)])
def test_mx_quantize_both_matches_the_two_single_passes(R, C):
    from torchtune_b200.ops._cuda import mx_quantize, mx_quantize_both

    x = _rand(R, C, seed=31, scale=3.0)
    x[5, :] = 0
    (q, sf), (qt, sft) = mx_quantize_both(x)
    q1, sf1 = mx_quantize(x)
    qt1, sft1 = mx_quantize(x, transpose=True)
    assert torch.equal(q, q1) and torch.equal(sf, sf1) and torch.equal(qt, qt1) and torch.equal(sft, sft1)


def test_out_of_range_user_indices_are_replaced_and_counted(monkeypatch):
    """Token ids, labels and positions outside their tables never reach an address computation: row 0 / an ignored row / position 0
    stand in, the event is counted, and TTB_DEBUG_BOUNDS=1 turns the count into an exception at the next device check."""
    from torchtune_b200.ops import _lib

    _lib.index_violations()  # clear
    table = _rand(64, 128, seed=1)
    ids = torch.tensor([[3, 64, -1, 5]], device="cuda")
    out = ops.embedding(ids, table)
    assert torch.equal(out[0, 1], table[0]) and torch.equal(out[0, 2], table[0]) and torch.equal(out[0, 0], table[3])
    assert _lib.index_violations() == 2
    hidden, w = _rand(8, 256, seed=2), _rand(128, 256, seed=3, scale=0.05)
    labels = torch.tensor([1, 2, 128, -5, -100, 7, 0, 127], device="cuda")
    loss_sum, n_valid = ops.linear_cross_entropy(hidden, w, labels, num_chunks=1)
    ref_labels = labels.clone()
    ref_labels[2:4] = -100
    want, _ = ops.linear_cross_entropy(hidden, w, ref_labels, num_chunks=1)
    assert torch.isfinite(loss_sum) and torch.allclose(loss_sum.float(), want.float(), rtol=1e-3)
    assert _lib.index_violations() == 2
    monkeypatch.setenv("TTB_DEBUG_BOUNDS", "1")
    _lib.err_word(torch.device("cuda"))
    ops.embedding(ids, table)
    with pytest.raises(_lib.KernelError, match="out-of-range"):
        _lib.check_device_errors()
    _lib.check_device_errors()  # the count was cleared by the failed check


@pytest.mark.parametrize("kind", ["forward", "reverse", "symmetric"])
def test_kd_divergence_kernel_matches_fp32_statement(kind):
    from torchtune_b200.modules.loss import ForwardKLLoss, ReverseKLLoss, SymmetricKLLoss

    loss = {"forward": ForwardKLLoss(), "reverse": ReverseKLLoss(), "symmetric": SymmetricKLLoss(sym_kd_ratio=0.3)}[kind]
    rows, V = 37, 1000
    student = _rand(rows, V, seed=41, scale=2.0).requires_grad_()
    teacher = _rand(rows, V, seed=42, scale=2.0)
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::5] = -100
    for normalize in (True, False):
        student.grad = None
        got = loss(student, teacher, labels, normalize=normalize)
        got.backward()
        s32 = student.detach().float().requires_grad_()
        want = loss(s32, teacher.float(), labels, normalize=normalize)  # fp32 inputs take the PyTorch statement
        want.backward()
        assert abs(got.item() - want.item()) < 2e-3 * max(1.0, abs(want.item())), (kind, got.item(), want.item())
        _close(student.grad, s32.grad, 2e-2, 2e-2 * s32.grad.abs().max().item(), f"kd {kind} grad")
        assert (student.grad[::5] == 0).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("top_k", [None, 1, 50, 300])
def test_sampling_kernel_matches_the_eager_statement(dtype, top_k):
    from torchtune_b200 import generation

    g = torch.Generator(device="cuda").manual_seed(7)
    logits = (torch.randn(6, 4099, generator=g, device="cuda") * 3).to(dtype)
    logits[0, 17] = logits[0].max() + 5  # a dominant token
    u = torch.rand(6, 4099, generator=g, device="cuda")
    q = -torch.log(torch.clamp(1.0 - u, min=1e-7))
    got = generation.sample(logits.clone(), temperature=0.7, top_k=top_k, q=q)
    assert got.shape == (6, 1) and got.dtype == torch.int32
    # the eager statement in fp32 on the same scaled logits (bf16 logits are divided in bf16, as the eager statement does)
    t = (logits / 0.7).float()
    if top_k is not None:
        kth = torch.topk(t, top_k).values[:, -1:]
        t = torch.where(t < kth, torch.full_like(t, float("-inf")), t)
    race = torch.softmax(t, dim=-1) / q
    picked = race.gather(1, got.long())
    assert (picked >= race.max(-1, keepdim=True).values * (1 - 1e-4)).all()  # the winner of the race, up to fp32 rounding of near-ties
    assert torch.isfinite(t.gather(1, got.long())).all()  # always a kept column
    with ops.use_reference_ops():
        want = generation.sample(logits.clone(), temperature=0.7, top_k=top_k, q=q)
    assert (got.long() == want.long()).float().mean() >= (1.0 if dtype == torch.float32 else 0.5)
    if top_k == 1:
        assert torch.equal(got.long(), logits.float().argmax(-1, keepdim=True))


@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_logits_to_logprobs_fused_matches_fp32(temperature):
    from torchtune_b200 import rlhf

    logits = _rand(3, 17, 2048, seed=51, scale=2.0).requires_grad_()
    tokens = torch.randint(0, 2048, (3, 17), device="cuda")
    got = rlhf.logits_to_logprobs(logits, tokens, temperature)
    assert got.dtype == torch.float32 and got.shape == (3, 17)
    w = torch.randn(3, 17, device="cuda")
    (got * w).sum().backward()
    l32 = logits.detach().float().requires_grad_()
    want = rlhf.logits_to_logprobs(l32, tokens, temperature)
    (want * w).sum().backward()
    _close(got, want, 2e-2, 2e-2, "logprobs")
    _close(logits.grad, l32.grad, 2e-2, 2e-2 * l32.grad.abs().max().item(), "logprobs grad")
    with torch.no_grad():
        _close(rlhf.logits_to_logprobs(logits, tokens, temperature), want, 2e-2, 2e-2, "logprobs (no grad)")


@pytest.mark.parametrize("M,N,K", [(8192, 4096, 1024), (4100, 6152, 512), (256, 512, 256)])  # the last one is too small for the CTA-pair kernel
def test_linear_residual_adds_in_the_epilogue(M, N, K):
    x = _rand(M, K, seed=61, scale=0.5).requires_grad_()
    w = _rand(N, K, seed=62, scale=0.05).requires_grad_()
    bias = _rand(N, seed=63, scale=0.2).requires_grad_()
    res = _rand(M, N, seed=64).requires_grad_()
    y = ops.linear_residual(x, w, bias, res)
    gy = _rand(M, N, seed=65)
    y.backward(gy)
    xr, wr, br, rr = (t.detach().float().requires_grad_() for t in (x, w, bias, res))
    yr = torch.nn.functional.linear(xr, wr, br) + rr
    yr.backward(gy.float())
    _close(y, yr, 2e-2, 2e-2, "linear_residual fwd")
    _close(res.grad, rr.grad, 0, 0, "linear_residual d residual")
    _close(x.grad, xr.grad, 2e-2, 5e-2, "linear_residual dx")
    _close(w.grad, wr.grad, 2e-2, 1.0, "linear_residual dw")


def test_decoder_layer_with_fused_residuals_matches_separate_additions(monkeypatch):
    from torchtune_b200.models.llama3_1 import llama3_1

    torch.manual_seed(0)
    model = llama3_1(vocab_size=512, num_layers=2, num_heads=8, num_kv_heads=2, embed_dim=1024, max_seq_len=2048, intermediate_dim=4096).cuda().bfloat16()
    tokens = torch.randint(0, 512, (4, 2048), device="cuda")

    def run():
        model.zero_grad(set_to_none=True)
        out = model(tokens)
        out.float().square().mean().backward()
        return out.detach().clone(), model.layers[0].attn.q_proj.weight.grad.detach().clone()

    assert model.layers[0]._fuse_residual_attn and model.layers[0]._fuse_residual_mlp
    fused_out, fused_grad = run()
    monkeypatch.setenv("TTB_FUSE_RESIDUAL", "0")
    plain_out, plain_grad = run()
    _close(fused_out, plain_out, 2e-2, 2e-2 * plain_out.abs().max().item(), "fused residual forward")
    _close(fused_grad, plain_grad, 5e-2, 5e-2 * plain_grad.abs().max().item(), "fused residual backward")
