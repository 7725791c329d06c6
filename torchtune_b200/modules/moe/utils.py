"""Switches for the expert matmul path (parity: torchtune/modules/moe/utils.py:13-40)."""
from __future__ import annotations

import torch

# With ``True`` the experts run as one batched computation over expert-sorted tokens; with
# ``False`` as an explicit per-expert loop (the layout needed by adapters and by debugging).
use_grouped_mm = True


def should_use_grouped_mm() -> bool:
    return use_grouped_mm


def expert_offsets(num_tokens_per_expert: torch.Tensor) -> torch.Tensor:
    """Exclusive prefix sums ``[E + 1]`` of the per-expert token counts."""
    counts = num_tokens_per_expert.to(torch.int64)
    return torch.cat([counts.new_zeros(1), counts.cumsum(0)])


def expert_load_imbalance(model: torch.nn.Module):
    """Mean over the MoE layers of ``max_e tokens(e) / mean_e tokens(e)`` for the most recent forward pass (1.0 = perfectly
    balanced routing); ``None`` for models without routers.  Counts are this rank's routed tokens."""
    ratios = []
    for m in model.modules():
        counts = getattr(m, "tokens_per_expert", None)
        if torch.is_tensor(counts) and counts.numel() > 0:
            c = counts.float()
            ratios.append(c.max() / c.mean().clamp_min(1e-9))
    return torch.stack(ratios).mean() if ratios else None
