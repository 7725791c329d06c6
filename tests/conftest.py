import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    # On a GPU box a bf16 CUDA operator that would leave the sm_100a kernels for a PyTorch statement raises instead of falling back,
    # so a test cannot pass on a silent fallback (TTB_STRICT=0 in the environment switches this off).
    os.environ.setdefault("TTB_STRICT", "1")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def tune_path():
    return str(ROOT / "torchtune_b200" / "_cli" / "tune.py")
