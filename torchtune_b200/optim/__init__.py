from .adamw import AdamW

__all__ = ["AdamW"]
