"""Seeding (parity: torchtune/training/seed.py:22-83)."""
from __future__ import annotations

import os
import random
from typing import Optional, Union

import numpy as np
import torch

from ..utils import get_logger, get_world_size_and_rank

_log = get_logger()


def _broadcast_int(value: int) -> int:
    if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
        return value
    backend = torch.distributed.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if "nccl" in str(backend) else torch.device("cpu")
    t = torch.tensor([value], dtype=torch.int64, device=dev)
    torch.distributed.broadcast(t, src=0)
    return int(t.item())


def set_seed(seed: Optional[int] = None, debug_mode: Union[str, int, None] = None) -> int:
    """Seed python, numpy and torch.  A missing seed is drawn on rank 0 and broadcast;
    every rank then uses ``seed + rank`` so dropout/shuffling differ across ranks.
    ``debug_mode`` (``default``/``warn``/``error`` or 0/1/2) switches on deterministic
    algorithms.  Returns the rank-local seed."""
    world, rank = get_world_size_and_rank()
    max_val, min_val = np.iinfo(np.uint32).max - world + 1, np.iinfo(np.uint32).min
    if seed is None:
        seed = _broadcast_int(int(torch.randint(min_val, max_val, (1,)).item()))
    if seed != 0 or world > 1:
        pass
    if seed < min_val or seed > max_val:
        raise ValueError(f"Invalid seed value provided: {seed}. Value must be in the range [{min_val}, {max_val}]")
    local = seed + rank
    if rank == 0:
        _log.debug(f"Setting manual seed to local seed {local}. Local seed is seed + rank = {seed} + {rank}")
    torch.manual_seed(local)
    np.random.seed(local)
    random.seed(local)
    if debug_mode is not None:
        _log.debug(f"Setting deterministic debug mode to {debug_mode}")
        torch.set_deterministic_debug_mode(debug_mode)
        deterministic = torch.get_deterministic_debug_mode() != 0
        torch.backends.cudnn.deterministic = deterministic
        torch.backends.cudnn.benchmark = not deterministic
        if deterministic:
            os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    return local
