from .adamw import AdamW
from .adamw8bit import AdamW8bit

__all__ = ["AdamW", "AdamW8bit"]
