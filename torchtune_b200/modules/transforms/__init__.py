from ._transforms import Transform, VisionCrossAttentionMask

__all__ = ["Transform", "VisionCrossAttentionMask"]
