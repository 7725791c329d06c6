"""Exceptions raised by the config layer (parity: torchtune/config/_errors.py:8-33)."""
from typing import List


class InstantiationError(Exception):
    """A ``_component_`` node could not be turned into an object."""


class ConfigError(Exception):
    """Aggregates every signature mismatch found while validating a config."""

    def __init__(self, errors: List[Exception]):
        super().__init__()
        self.errors = list(errors)

    def __str__(self) -> str:
        lines = [f"Config is not well-formed, found the following errors ({len(self.errors)}):"]
        lines += [f"  - {e}" for e in self.errors]
        return "\n".join(lines)
