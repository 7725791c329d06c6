"""The allocation-free RMSNorm backward (``ttb_rmsnorm_bwd_noalloc``), called through its
exported C symbol, must reproduce the regular entry point (``ttb_rmsnorm_bwd``, which uses a
caller-provided scratch buffer) — twice in a row, because the second call reuses the
library's built-in scratch array with the first call's contents still in it.

Collected last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rows, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, D, generator=g, device="cuda").bfloat16()
    dy = torch.randn(rows, D, generator=g, device="cuda").bfloat16()
    scale = (1 + 0.1 * torch.randn(D, generator=g, device="cuda")).bfloat16()
    return x, dy, scale


def _run_both(L, rows, D, seed):
    from torchtune_b200.ops._lib import check, stream_ptr

    x, dy, scale = _inputs(rows, D, seed)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
    check(L.ttb_rmsnorm_fwd(x.data_ptr(), scale.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, D, 1e-5, stream_ptr()), "fwd")

    # existing entry point: caller-allocated partial sums, summed by the caller
    n_part = L.ttb_rmsnorm_bwd_partials(rows)
    partial = torch.empty(n_part, D, dtype=torch.float32, device="cuda")
    dx_ref = torch.empty_like(x)
    check(L.ttb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(), partial.data_ptr(), rows, D, stream_ptr()), "bwd")
    dscale_ref = partial.sum(0)

    # new entry point: outputs only, no scratch argument
    dx = torch.empty_like(x)
    dscale = torch.empty(D, dtype=torch.float32, device="cuda")
    rc = L.ttb_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dscale.data_ptr(), rows, D, stream_ptr())
    assert rc == 0, rc
    torch.cuda.synchronize()
    torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dscale, dscale_ref, rtol=2e-2, atol=2e-2 * rows**0.5)


def test_noalloc_matches_regular_entry_point_twice():
    from torchtune_b200.ops._lib import lib

    L = lib()
    fn = L.ttb_rmsnorm_bwd_noalloc
    vp = ctypes.c_void_p
    fn.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, vp]
    fn.restype = ctypes.c_int
    # two calls in a row with different shapes and data: stale scratch must not leak through
    _run_both(L, 1000, 4096, seed=1)
    _run_both(L, 37, 256, seed=2)
    _run_both(L, 300, 8192, seed=3)


def test_noalloc_without_scale_matches_regular_entry_point():
    """Weight-less norm: no partial sums, no finalize pass, ``dscale`` may be null."""
    from torchtune_b200.ops._lib import check, lib, stream_ptr

    L = lib()
    fn = L.ttb_rmsnorm_bwd_noalloc
    vp = ctypes.c_void_p
    fn.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, vp]
    fn.restype = ctypes.c_int
    for rows, D, seed in ((513, 1024, 4), (64, 4096, 5)):
        x, dy, _ = _inputs(rows, D, seed)
        y = torch.empty_like(x)
        rstd = torch.empty(rows, dtype=torch.float32, device="cuda")
        check(L.ttb_rmsnorm_fwd(x.data_ptr(), None, y.data_ptr(), rstd.data_ptr(), rows, D, 1e-5, stream_ptr()), "fwd")
        dx_ref = torch.empty_like(x)
        check(L.ttb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), None, rstd.data_ptr(), dx_ref.data_ptr(), None, rows, D, stream_ptr()), "bwd")
        dx = torch.empty_like(x)
        assert fn(dy.data_ptr(), x.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), None, rows, D, stream_ptr()) == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)


def test_noalloc_rejects_oversized_rows():
    from torchtune_b200.ops._lib import lib

    L = lib()
    fn = L.ttb_rmsnorm_bwd_noalloc
    vp = ctypes.c_void_p
    fn.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, vp]
    fn.restype = ctypes.c_int
    t = torch.zeros(8, device="cuda")
    assert fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4, 16384, None) == -3
    assert fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4, 100, None) == -1
