"""AdamW with one-byte moments: follows fp32 AdamW on a regression problem, keeps a quarter of the state, survives a state-dict round
trip, and stands in for the 8-bit optimizers of packages that are not installed."""
import pytest
import torch

from torchtune_b200 import config
from torchtune_b200.ops import reference as ref
from torchtune_b200.optim import AdamW8bit


def _problem(seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(256, 64, generator=g)
    w_true = torch.randn(64, 96, generator=g)
    y = x @ w_true
    w0 = torch.randn(64, 96, generator=g) * 0.1
    return x, y, w0


def _train(opt_cls, steps=200, **kw):
    x, y, w0 = _problem()
    w = torch.nn.Parameter(w0.clone())
    b = torch.nn.Parameter(torch.zeros(96))
    opt = opt_cls([w, b], lr=1e-2, weight_decay=0.01, **kw)
    losses = []
    for _ in range(steps):
        loss = ((x @ w + b - y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return w.detach(), losses, opt


def test_follows_fp32_adamw():
    w_ref, l_ref, _ = _train(torch.optim.AdamW, steps=600)
    w_q, l_q, opt = _train(AdamW8bit, steps=600)
    assert l_q[-1] < 1e-3 * l_q[0]
    assert all(abs(a - b) < 0.1 * b for a, b in zip(l_q[::50], l_ref[::50]))  # the whole curve, not only its end
    assert (w_q - w_ref).norm() / w_ref.norm() < 0.02
    # the weight (6144 elements) is coded; the bias (96) keeps fp32 moments
    kinds = [sorted(k for k in st if k != "step") for st in opt.state.values()]
    assert kinds == [["exp_avg_q", "exp_avg_scale", "exp_avg_sq_q", "exp_avg_sq_scale"], ["exp_avg", "exp_avg_sq"]]
    assert opt.state_bytes() == 6144 * 2 + 24 * 8 + 96 * 8


def test_codes_round_trip_within_one_step_of_the_code():
    torch.manual_seed(0)
    n = 1000  # not a multiple of the block
    m = torch.randn(n) * torch.logspace(-4, 0, n)
    v = (torch.randn(n) * torch.logspace(-6, 0, n)) ** 2
    p, g = torch.zeros(n), torch.zeros(n)
    mq, vq = torch.zeros(n, dtype=torch.int8), torch.zeros(n, dtype=torch.uint8)
    ms, vs = torch.zeros(4), torch.zeros(4)
    # one step with beta = 0 and unit gradient scale stores g and g² as the moments
    ref.adamw8bit_step(p, m.clone(), mq, vq, ms, vs, step=1, lr=0.0, beta1=0.0, beta2=0.0, eps=1e-8, weight_decay=0.0)
    m2, v2 = ref.adamw8bit_decode(mq, vq, ms, vs, n)
    block_max = ms[torch.arange(n) // 256]
    # square-root companding: the error of an entry is at most one code step at its own magnitude, 2·sqrt(|m|·max)/127 (+ rounding)
    assert ((m2 - m).abs() <= (m.abs() * block_max).sqrt() / 127 + block_max / 127**2 + 1e-12).all()
    vmax = vs[torch.arange(n) // 256]
    true_v = m * m
    assert ((v2.sqrt().sqrt() - true_v.sqrt().sqrt()).abs() <= vmax.sqrt().sqrt() / 255 * 0.51 + 1e-12).all()


def test_state_dict_round_trip_continues_identically():
    x, y, w0 = _problem()

    def make():
        w = torch.nn.Parameter(w0.clone())
        return w, AdamW8bit([w], lr=1e-2)

    def run(w, opt, steps):
        for _ in range(steps):
            loss = ((x @ w - y) ** 2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()

    w1, o1 = make()
    run(w1, o1, 10)
    w2, o2 = make()
    run(w2, o2, 5)
    w3, o3 = make()
    with torch.no_grad():
        w3.copy_(w2)
    o3.load_state_dict(o2.state_dict())
    run(w3, o3, 5)
    assert torch.equal(w3, w1)
    assert o3.state[w3]["exp_avg_q"].dtype == torch.int8 and o3.state[w3]["exp_avg_sq_q"].dtype == torch.uint8


def test_stands_in_for_packages_that_are_not_installed():
    for name in ("bitsandbytes.optim.PagedAdamW8bit", "torchao.optim.AdamW8bit"):
        module = name.split(".")[0]
        try:
            __import__(module)
            pytest.skip(f"{module} is installed here")
        except ImportError:
            pass
        cfg = config.OmegaConf.create({"optimizer": {"_component_": name, "lr": 2e-5}})
        opt = config.instantiate(cfg.optimizer, [torch.nn.Parameter(torch.zeros(8))])
        assert isinstance(opt, AdamW8bit) and opt.param_groups[0]["lr"] == 2e-5
    with pytest.raises(config.InstantiationError if hasattr(config, "InstantiationError") else Exception):
        config.instantiate(config.OmegaConf.create({"_component_": "bitsandbytes.optim.SomethingElse"}))


def test_host_offload_wrapper_of_an_absent_package_builds_the_inner_optimizer_on_the_device():
    try:
        import torchao  # noqa: F401

        pytest.skip("torchao is installed here")
    except ImportError:
        pass
    cfg = config.OmegaConf.create({"optimizer": {"_component_": "torchao.optim.CPUOffloadOptimizer", "optimizer_class": "torch.optim.AdamW", "offload_gradients": True, "lr": 3e-4}})
    p = torch.nn.Parameter(torch.zeros(4))
    opt = config.instantiate(cfg.optimizer, [p])
    assert type(opt) is torch.optim.AdamW and opt.param_groups[0]["lr"] == 3e-4
