"""Shared data constants (parity: torchtune/data/_common.py)."""
from typing import Dict, List, Union

import torch

CROSS_ENTROPY_IGNORE_IDX = -100
PACK_TYPE = Dict[str, Union[torch.Tensor, List[int]]]
