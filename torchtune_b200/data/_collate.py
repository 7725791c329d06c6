"""Batch collation (parity: torchtune/data/_collate.py:15-725)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F
from torch.nn.utils.rnn import pad_sequence

from ..ops.mask import AttentionMask
from ._common import CROSS_ENTROPY_IGNORE_IDX, PACK_TYPE


def _as_tensor(x) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.tensor(x)


def left_pad_sequence(sequences: List[torch.Tensor], batch_first: bool = False, padding_value: float = 0) -> torch.Tensor:
    """Pad variable-length sequences on the **left**."""
    flipped = pad_sequence([s.flip(0) for s in sequences], batch_first=batch_first, padding_value=padding_value)
    return flipped.flip(int(batch_first))


def padded_collate(
    batch: List[Dict[str, List[int]]],
    *,
    pad_direction: str,
    keys_to_pad: List[str],
    padding_idx: Union[int, Dict[str, int]],
) -> Dict[str, torch.Tensor]:
    """Pad the listed keys of every sample to the batch max (left or right); other keys
    are stacked into tensors unchanged."""
    if pad_direction not in ("left", "right"):
        raise ValueError(f"pad_direction should be one of 'left' or 'right' but found {pad_direction}")
    if not isinstance(padding_idx, int):
        if set(padding_idx) != set(keys_to_pad):
            raise ValueError(f"padding_idx was provided as a dictionary, but the keys ({padding_idx.keys()}) do not match keys_to_pad ({keys_to_pad})")
    if not keys_to_pad:
        raise ValueError("keys_to_pad must be a non-empty list")
    if any(k not in batch[0] for k in keys_to_pad):
        raise ValueError(f"keys_to_pad ({keys_to_pad}) must be a subset of the batch keys ({batch[0].keys()})")
    out: Dict[str, torch.Tensor] = {}
    for k in batch[0]:
        if k in keys_to_pad:
            pad = padding_idx if isinstance(padding_idx, int) else padding_idx[k]
            seqs = [_as_tensor(x[k]) for x in batch]
            out[k] = left_pad_sequence(seqs, True, pad) if pad_direction == "left" else pad_sequence(seqs, True, pad)
        else:
            out[k] = torch.tensor([x[k] for x in batch])
    return out


def padded_collate_sft(
    batch: List[Dict[str, Any]],
    padding_idx: int = 0,
    ignore_idx: int = CROSS_ENTROPY_IGNORE_IDX,
    pad_to_multiple_of: int = 1,
    stack_on_new_dim: bool = False,
    cp_degree: int = 1,
) -> Dict[str, torch.Tensor]:
    """Right-pad ``tokens`` with ``padding_idx`` and ``labels`` with ``ignore_idx`` to the
    batch max.  With ``pad_to_multiple_of > 1`` the amount ``m - len % m`` is appended
    (a full extra multiple when the length already divides — kept for parity).
    ``cp_degree > 1`` adds explicit ``input_pos``."""
    tokens = pad_sequence([_as_tensor(x["tokens"]) for x in batch], batch_first=True, padding_value=padding_idx)
    labels = pad_sequence([_as_tensor(x["labels"]) for x in batch], batch_first=True, padding_value=ignore_idx)
    width = max(tokens.shape[-1], labels.shape[-1])
    tokens = F.pad(tokens, (0, width - tokens.shape[-1]), value=padding_idx)
    labels = F.pad(labels, (0, width - labels.shape[-1]), value=ignore_idx)
    if pad_to_multiple_of > 1:
        extra = pad_to_multiple_of - (width % pad_to_multiple_of)
        tokens = F.pad(tokens, (0, extra), value=padding_idx)
        labels = F.pad(labels, (0, extra), value=ignore_idx)
    out: Dict[str, Any] = {"tokens": tokens.long(), "labels": labels.long()}
    if cp_degree > 1:
        b, n = tokens.shape
        out["input_pos"] = torch.arange(n, dtype=torch.long).repeat(b, 1)
    if "encoder_input" in batch[0]:
        enc = _stack_encoder_input([x["encoder_input"] for x in batch], new_dim=stack_on_new_dim)
        if enc:
            out["encoder_input"] = enc
    return out


def _stack_encoder_input(items: List[Dict[str, Any]], new_dim: bool = False) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for key in items[0]:
        vals = [d[key] for d in items]
        if isinstance(vals[0], torch.Tensor):
            out[key] = torch.stack(vals) if new_dim else torch.cat(vals, dim=0)
        elif isinstance(vals[0], dict):
            out[key] = _stack_encoder_input(vals, new_dim)
        elif isinstance(vals[0], (list, tuple)) and vals[0] and isinstance(vals[0][0], torch.Tensor):
            flat = [t for v in vals for t in v]
            out[key] = torch.stack(flat) if new_dim else torch.cat(flat, dim=0)
    return out


def padded_collate_packed(batch: List[PACK_TYPE]) -> Dict[str, Any]:
    """Stack already-packed samples and describe their block-causal structure: the
    returned ``mask`` is an :class:`AttentionMask` carrying one document id per token."""
    tokens = torch.stack([_as_tensor(x["tokens"]) for x in batch])
    labels = torch.stack([_as_tensor(x["labels"]) for x in batch])
    input_pos = torch.stack([_as_tensor(x["input_pos"]) for x in batch])
    mask = AttentionMask.from_seq_lens([_as_tensor(x["seq_lens"]) for x in batch], max_len=tokens.shape[1])
    return {"tokens": tokens, "labels": labels, "input_pos": input_pos, "mask": mask}


def padded_collate_dpo(
    batch: List[Dict[str, List[int]]], padding_idx: int = 0, ignore_idx: int = CROSS_ENTROPY_IGNORE_IDX
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Concatenate chosen then rejected sequences along the batch dimension, right-padded:
    returns ``(input_ids [2B, L], labels [2B, L])``."""
    ids = [_as_tensor(x["chosen_input_ids"]) for x in batch] + [_as_tensor(x["rejected_input_ids"]) for x in batch]
    lbl = [_as_tensor(x["chosen_labels"]) for x in batch] + [_as_tensor(x["rejected_labels"]) for x in batch]
    for a, b in zip(ids, lbl):
        assert len(a) == len(b)
    return (
        pad_sequence(ids, batch_first=True, padding_value=padding_idx),
        pad_sequence(lbl, batch_first=True, padding_value=ignore_idx),
    )


def padded_collate_tiled_images_and_mask(
    batch: List[Dict[str, Any]],
    padding_idx: int = 0,
    ignore_idx: int = CROSS_ENTROPY_IGNORE_IDX,
    pad_direction: str = "right",
    pad_max_tiles: Optional[int] = None,
    pad_max_images: Optional[int] = None,
    pad_to_multiple_of: int = 1,
) -> Dict[str, Any]:
    """Collate text plus tiled images for cross-attention vision models.

    Text is padded like :func:`padded_collate_sft` (left padding allowed for inference);
    every image is padded to the max tile count, every sample to the max image count, and
    each per-image cross-attention mask ``[text_len, tiles*tokens_per_tile]`` is padded
    and concatenated along the image-token axis."""
    if pad_direction not in ("left", "right"):
        raise ValueError(f"pad_direction should be one of 'left' or 'right' but found {pad_direction}")
    text_only = [{k: v for k, v in s.items() if k in ("tokens", "labels")} for s in batch]
    if pad_direction == "right":
        text = padded_collate_sft(text_only, padding_idx, ignore_idx, pad_to_multiple_of=pad_to_multiple_of)
    else:
        if "labels" in batch[0]:
            raise ValueError("labels are not supported with left padding (inference only)")
        text = {"tokens": left_pad_sequence([_as_tensor(s["tokens"]) for s in batch], True, padding_idx)}
    max_seq = text["tokens"].shape[-1]
    bsz = len(batch)

    max_tiles = max((img.shape[0] for s in batch for img in s["encoder_input"]["images"]), default=1)
    if pad_max_tiles is not None:
        if pad_max_tiles < max_tiles:
            raise ValueError(f"More tiles in image {max_tiles}, than pad_max_tiles {pad_max_tiles}")
        max_tiles = pad_max_tiles
    first_img = next(img for s in batch for img in s["encoder_input"]["images"])
    _, c, h, w = first_img.shape
    first_mask = next(m for s in batch for m in s["encoder_mask"])
    tokens_per_tile = first_mask.shape[1] // first_img.shape[0] if first_img.shape[0] else first_mask.shape[1]
    max_images = max(len(s["encoder_input"]["images"]) for s in batch)
    if pad_max_images is not None:
        max_images = max(max_images, pad_max_images)

    images = torch.zeros(bsz, max_images, max_tiles, c, h, w, dtype=first_img.dtype)
    ratios = torch.ones(bsz, max_images, 2, dtype=torch.long)
    masks = torch.zeros(bsz, max_seq, max_images * max_tiles * tokens_per_tile, dtype=torch.bool)
    for i, s in enumerate(batch):
        seq = len(s["tokens"])
        off = max_seq - seq if pad_direction == "left" else 0
        for j, (img, ar, m) in enumerate(zip(s["encoder_input"]["images"], s["encoder_input"]["aspect_ratio"], s["encoder_mask"])):
            nt = img.shape[0]
            images[i, j, :nt] = img
            ratios[i, j] = _as_tensor(ar)
            start = j * max_tiles * tokens_per_tile
            masks[i, off : off + m.shape[0], start : start + m.shape[1]] = m.bool()
    out = dict(text)
    out["encoder_input"] = {"images": images, "aspect_ratio": ratios}
    out["encoder_mask"] = masks
    return out
