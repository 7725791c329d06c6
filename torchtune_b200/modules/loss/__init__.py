from .ce_chunked_output_loss import CEWithChunkedOutputLoss
from .cross_entropy_loss import LinearCrossEntropyLoss
from .kd_losses import (
    ForwardKLLoss,
    ForwardKLWithChunkedOutputLoss,
    ReverseKLLoss,
    ReverseKLWithChunkedOutputLoss,
    SymmetricKLLoss,
    SymmetricKLWithChunkedOutputLoss,
)
from .loss_types import RLLoss, SFTLoss

__all__ = [
    "CEWithChunkedOutputLoss",
    "LinearCrossEntropyLoss",
    "ForwardKLLoss",
    "ForwardKLWithChunkedOutputLoss",
    "ReverseKLLoss",
    "ReverseKLWithChunkedOutputLoss",
    "SymmetricKLLoss",
    "SymmetricKLWithChunkedOutputLoss",
    "RLLoss",
    "SFTLoss",
]
