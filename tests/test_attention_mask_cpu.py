"""Host-side mask descriptions handed to the attention kernels: per-row visible ranges of a boolean mask, per-query lower
bounds of the structured masks."""
import torch

from torchtune_b200.ops import AttentionMask
from torchtune_b200.ops._cuda_attention import dense_mask_bounds, lower_bounds, unsupported_reason


def test_dense_mask_bounds_first_and_last_visible_key():
    g = torch.Generator().manual_seed(0)
    m = torch.rand(2, 7, 13, generator=g) < 0.3
    m[0, 3] = False  # a row that sees nothing
    kmask, lo, hi = dense_mask_bounds(m, 2, 7, 13)
    assert kmask.dtype == torch.uint8 and kmask.shape == (2, 7, 13) and torch.equal(kmask.bool(), m)
    for b in range(2):
        for r in range(7):
            idx = m[b, r].nonzero().flatten()
            want = (13, -1) if idx.numel() == 0 else (int(idx[0]), int(idx[-1]))
            assert (int(lo[b, r]), int(hi[b, r])) == want
    # broadcastable forms: [1, s, sk] and [b, 1, s, sk]
    k2, lo2, _ = dense_mask_bounds(m[:1], 2, 7, 13)
    assert torch.equal(k2[1], k2[0]) and torch.equal(lo2[1], lo2[0])
    k3, _, _ = dense_mask_bounds(m.unsqueeze(1), 2, 7, 13)
    assert torch.equal(k3, kmask)


def test_lower_bounds_and_unsupported_cases():
    mask = AttentionMask.from_seq_lens([[3, 5]])
    lo = lower_bounds(mask, 1, 8, torch.device("cpu"))
    assert lo.tolist() == [[0, 0, 0, 3, 3, 3, 3, 3]]
    lo = lower_bounds(AttentionMask(causal=True, window=3), 1, 6, torch.device("cpu"))
    assert lo.tolist() == [[0, 0, 0, 1, 2, 3]]
    q, k = torch.zeros(1, 4, 8, 64), torch.zeros(1, 9, 2, 64)
    assert unsupported_reason(q, k, AttentionMask(causal=False)) is None  # cross-attention lengths are fine
    assert unsupported_reason(q, k, AttentionMask(causal=True)) is None  # bottom-right aligned causal
    assert "different query and key lengths" in unsupported_reason(q, k, AttentionMask(causal=True, window=4))
    assert "per-head" in unsupported_reason(q, k, AttentionMask(causal=False, bool_mask=torch.ones(1, 8, 4, 9, dtype=torch.bool)))
    assert unsupported_reason(q, torch.zeros(1, 9, 3, 64), AttentionMask(causal=False)) is not None
