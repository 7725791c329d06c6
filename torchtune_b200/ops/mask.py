"""Structured attention-mask descriptor.

Instead of a dense ``[b, s, s]`` boolean tensor or a compiled block mask
(torchtune/modules/attention_utils.py:133-252), training masks are described by
a handful of fields the attention kernel evaluates per tile: causal flag,
per-token document id (sample packing), chunk size (Llama-4 local attention,
torchtune/models/llama4/_chunked_attention.py:20-57) and sliding window.  A
dense boolean mask remains available for inference paths.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional, Sequence

import torch


@dataclass
class AttentionMask:
    causal: bool = True
    doc_ids: Optional[torch.Tensor] = None  # [b, s] int32, equal ids may attend
    chunk: int = 0  # >0: positions attend only inside the same chunk of this size
    window: int = 0  # >0: key must be within this many positions before the query
    bool_mask: Optional[torch.Tensor] = None  # dense [b, sq, skv], True = attend

    def to(self, device, non_blocking: bool = False) -> "AttentionMask":
        return replace(
            self,
            doc_ids=None if self.doc_ids is None else self.doc_ids.to(device, non_blocking=non_blocking),
            bool_mask=None if self.bool_mask is None else self.bool_mask.to(device, non_blocking=non_blocking),
        )

    def with_chunk(self, chunk: int) -> "AttentionMask":
        return replace(self, chunk=chunk)

    def dense(self, b: int, sq: int, skv: int, device) -> Optional[torch.Tensor]:
        """Materialise ``[b, sq, skv]`` booleans (tests and fallbacks only)."""
        if self.bool_mask is not None:
            return self.bool_mask
        from .reference import dense_mask

        m = dense_mask(b, sq, skv, device, self.causal, self.doc_ids, self.chunk, self.window)
        return None if m is None else m.squeeze(1)

    @staticmethod
    def from_seq_lens(seq_lens: Sequence[torch.Tensor] | Sequence[Sequence[int]], max_len: Optional[int] = None) -> "AttentionMask":
        """Block-causal mask for packed samples: one row of document lengths per batch
        entry; a trailing remainder up to ``max_len`` becomes its own document."""
        rows: List[torch.Tensor] = []
        for lens in seq_lens:
            lens_t = torch.as_tensor(lens, dtype=torch.long)
            ids = torch.repeat_interleave(torch.arange(len(lens_t)), lens_t)
            if max_len is not None and ids.numel() < max_len:
                ids = torch.cat([ids, torch.full((max_len - ids.numel(),), len(lens_t), dtype=torch.long)])
            rows.append(ids)
        return AttentionMask(causal=True, doc_ids=torch.stack(rows).to(torch.int32))
