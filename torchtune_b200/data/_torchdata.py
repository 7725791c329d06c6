"""Guards for code that needs the optional ``torchdata`` package (parity: torchtune/data/_torchdata.py:34-58).

Nothing inside this package depends on ``torchdata``: the multi-dataset loader is
:class:`torchtune_b200.datasets.InterleavedDataset` over map-style datasets.  User code ported from the reference that builds
``torchdata.nodes`` graphs can keep its decorators."""
from __future__ import annotations

import functools
import importlib.util
from typing import Callable

_MIN_VERSION = "0.10.0"


def _installed() -> bool:
    if importlib.util.find_spec("torchdata") is None:
        return False
    try:
        import torchdata
        from packaging.version import Version

        return Version(getattr(torchdata, "__version__", "0")) >= Version(_MIN_VERSION) and importlib.util.find_spec("torchdata.nodes") is not None
    except Exception:
        return False


def assert_torchdata_installed() -> None:
    if not _installed():
        raise ImportError(f"torchdata is not installed, or the installed version is older than {_MIN_VERSION}: `pip install torchdata>={_MIN_VERSION}`")


def requires_torchdata(func: Callable) -> Callable:
    """Decorator: the wrapped function raises ``ImportError`` with installation advice when ``torchdata`` is missing."""

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        assert_torchdata_installed()
        return func(*args, **kwargs)

    return wrapper
