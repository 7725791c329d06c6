"""Version comparison helper (parity: torchtune/utils/_version.py:12-28)."""
import torch


def _key(v: str):
    core = v.split("+")[0]
    out = []
    for piece in core.split("."):
        digits = "".join(ch for ch in piece if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out)


def torch_version_ge(version: str) -> bool:
    """True when the installed torch is at least ``version``."""
    return _key(torch.__version__) >= _key(version)
