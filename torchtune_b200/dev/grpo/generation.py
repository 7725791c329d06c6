"""Rollout generation under the module path the reference uses (torchtune/dev/grpo/generation.py); the code lives in
:mod:`torchtune_b200.dev.rl.generation`."""
from ..rl.generation import generate

__all__ = ["generate"]
