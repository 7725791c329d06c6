"""Permutation indices that regroup expert-parallel all-to-all output by local expert, each
group padded to an alignment (parity: torchtune/modules/moe/indices.py:23-230).

After the dispatch all-to-all a rank holds, for each source rank ``r`` and each of its local
experts ``e``, a run of ``tokens_per_expert_group[r·E_local + e]`` rows, laid out rank-major.
The grouped GEMM wants them expert-major with every expert's block starting at a multiple of
``alignment``.  ``generate_permute_indices`` returns the gather indices (``-1`` = padding row),
the padded group sizes and their offsets.  The computation is a segmented prefix sum: one
kernel on CUDA (``csrc/moe.cu``, every output slot pulls its source index), tensor ops elsewhere.
"""
from __future__ import annotations

from typing import Tuple

import torch


def generate_permute_indices(tokens_per_expert_group: torch.Tensor, experts_per_rank: int, num_ranks: int, max_len: int, alignment: int, use_cpu: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if tokens_per_expert_group.is_cuda and not use_cpu and num_ranks * experts_per_rank <= 4096:
        from ...ops import cuda_ops_enabled

        if cuda_ops_enabled(tokens_per_expert_group):
            from ...ops._cuda import moe_permute_indices

            return moe_permute_indices(tokens_per_expert_group, experts_per_rank, num_ranks, max_len, alignment)
    dev = torch.device("cpu") if use_cpu else tokens_per_expert_group.device
    counts = tokens_per_expert_group.to(dev, torch.int64).view(num_ranks, experts_per_rank)
    # where each (rank, expert) run starts in the rank-major input
    in_start = (counts.reshape(-1).cumsum(0) - counts.reshape(-1)).view(num_ranks, experts_per_rank)
    per_expert = counts.sum(0)
    m_sizes = torch.clamp_min((per_expert + alignment - 1) // alignment * alignment, alignment)
    m_offsets = m_sizes.cumsum(0)
    out_start = m_offsets - m_sizes
    # position of run (r, e) inside expert e's block = tokens of ranks < r for that expert
    within = counts.cumsum(0) - counts
    run_out_start = out_start.unsqueeze(0) + within  # [R, E]
    permuted = torch.full((max_len,), -1, dtype=torch.int32, device=dev)
    total = int(counts.sum())
    if total:
        run_len = counts.reshape(-1)
        run_id = torch.repeat_interleave(torch.arange(run_len.numel(), device=dev), run_len)
        pos_in_run = torch.arange(total, device=dev) - torch.repeat_interleave(run_len.cumsum(0) - run_len, run_len)
        src = in_start.reshape(-1)[run_id] + pos_in_run
        dst = run_out_start.reshape(-1)[run_id] + pos_in_run
        keep = dst < max_len
        permuted[dst[keep]] = src[keep].to(torch.int32)
    return permuted, m_sizes.to(torch.int32), m_offsets.to(torch.int32)


def fill_indices_cpu(tokens_per_expert_group: torch.Tensor, start_index_values: torch.Tensor, write_offsets: torch.Tensor, experts_per_rank: int, num_ranks: int, max_len: int) -> torch.Tensor:
    """Loop form of the same fill, kept as the oracle for tests."""
    out = torch.full((max_len,), -1, dtype=torch.int32)
    for e in range(experts_per_rank):
        w = int(write_offsets[e])
        for r in range(num_ranks):
            i = r * experts_per_rank + e
            n, s = int(tokens_per_expert_group[i]), int(start_index_values[i])
            n = max(min(n, max_len - w), 0)
            if n:
                out[w : w + n] = torch.arange(s, s + n, dtype=torch.int32)
            w += n
    return out


def fill_indices_wrapper(tokens_per_expert_group: torch.Tensor, start_index_values: torch.Tensor, write_offsets: torch.Tensor, experts_per_rank: int, num_ranks: int, total_size: int,
                         block_size: int = 128, max_blocks: int = 1024) -> torch.Tensor:
    """Fill the permutation from precomputed run starts and per-expert write offsets, on the tensors' own device and without a
    host loop (the reference launches a Triton kernel here, torchtune/modules/moe/indices.py:75-108; ``block_size`` and
    ``max_blocks`` are its launch parameters and have no meaning for this vectorised form).  Run ``(r, e)`` — ``tokens[r·E + e]``
    consecutive source rows from ``start_index_values[r·E + e]`` — is written after the runs of lower ranks for the same expert,
    beginning at ``write_offsets[e]``; unwritten slots stay ``-1``."""
    dev = tokens_per_expert_group.device
    counts = tokens_per_expert_group.to(torch.int64).view(num_ranks, experts_per_rank)
    starts = start_index_values.to(torch.int64).view(num_ranks, experts_per_rank)
    dst0 = write_offsets.to(torch.int64).view(1, experts_per_rank) + (counts.cumsum(0) - counts)
    out = torch.full((total_size,), -1, dtype=torch.int32, device=dev)
    run_len = counts.reshape(-1)
    total = int(run_len.sum())
    if total:
        run_id = torch.repeat_interleave(torch.arange(run_len.numel(), device=dev), run_len)
        pos = torch.arange(total, device=dev) - torch.repeat_interleave(run_len.cumsum(0) - run_len, run_len)
        dst = dst0.reshape(-1)[run_id] + pos
        keep = dst < total_size
        out[dst[keep]] = (starts.reshape(-1)[run_id] + pos)[keep].to(torch.int32)
    return out
