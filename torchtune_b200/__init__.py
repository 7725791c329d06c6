"""B200-native LLM post-training framework.

PyTorch is the framework layer; hot operators are hand-written sm_100a CUDA
kernels (``torchtune_b200.ops``) and collectives are fused into them over
NVLink peer memory (``torchtune_b200.parallel``).
"""
import os

# Growable segments avoid fragmentation with per-layer gather buffers; must be
# set before the CUDA caching allocator initialises.
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

__version__ = "0.1.0"

from . import config, utils  # noqa: E402,F401
