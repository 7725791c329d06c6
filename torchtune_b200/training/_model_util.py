"""Model tweaks (parity: torchtune/training/_model_util.py:11-23)."""
import warnings

import torch


def disable_dropout(model: torch.nn.Module) -> None:
    """Zero every ``nn.Dropout`` probability (used for DPO/PPO reference behaviour)."""
    for m in model.modules():
        if isinstance(m, torch.nn.Dropout) and m.p != 0:
            warnings.warn(f"Found Dropout with value {m.p} in module {type(m).__name__}. Setting to zero.")
            m.p = 0
