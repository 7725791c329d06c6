"""Inference-side half of the weight synchronisation (parity: torchtune/dev/rl/workers/weight_updaters/weight_updater.py:14-59)."""
from __future__ import annotations

from torch import nn

from .parameter_servers import ParameterServer


class WeightUpdateReceiver:
    def __init__(self, server: ParameterServer, model: nn.Module):
        self.server, self.model = server, model
        self.version = 0

    def maybe_update(self) -> bool:
        """Load newer weights into the model if the server has any; returns whether it did."""
        got = self.server.fetch(self.version)
        if got is None:
            return False
        self.version, weights = got
        self.model.load_state_dict(weights, strict=False)
        return True
