"""Tensor bundles of the GRPO recipes (parity: torchtune/dev/rl/types.py:13-64); shared with the synchronous recipe."""
from ..grpo.types import GRPOStats, GRPOTrajectory

__all__ = ["GRPOStats", "GRPOTrajectory"]
