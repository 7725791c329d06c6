"""Logging helpers (parity: torchtune/utils/_logging.py:18-147)."""
from __future__ import annotations

import functools
import logging
import warnings
from typing import Callable, Optional, TypeVar

T = TypeVar("T")


def get_logger(level: Optional[str] = None) -> logging.Logger:
    """Package logger with a stream handler attached exactly once."""
    logger = logging.getLogger(__name__.split(".")[0])
    if not logger.hasHandlers():
        logger.addHandler(logging.StreamHandler())
    if level is not None:
        logger.setLevel(getattr(logging, level.upper()))
    return logger


def log_rank_zero(logger: logging.Logger, msg: str, level: int = logging.INFO) -> None:
    from ._device import get_world_size_and_rank

    if get_world_size_and_rank()[1] == 0:
        logger.log(level, msg, stacklevel=2)


@functools.lru_cache(None)
def log_once(logger: logging.Logger, msg: str, level: int = logging.INFO) -> None:
    """Emit ``msg`` a single time per process (and only on rank zero)."""
    log_rank_zero(logger, msg, level)


def deprecated(msg: str = "") -> Callable[[T], T]:
    """Decorator that warns once when a class or function is used."""

    @functools.lru_cache(maxsize=1)
    def _warn(obj) -> None:
        warnings.warn(
            f"{obj.__name__} is deprecated and will be removed in future versions. {msg}",
            category=FutureWarning,
            stacklevel=3,
        )

    def decorator(obj):
        @functools.wraps(obj)
        def wrapper(*args, **kwargs):
            _warn(obj)
            return obj(*args, **kwargs)

        return wrapper

    return decorator


def deprecate_parameter(param_name: str, msg: str = "") -> Callable[[T], T]:
    """Decorator that warns (once) when the decorated callable is given the keyword argument ``param_name``."""

    @functools.lru_cache(maxsize=1)
    def _warn(obj) -> None:
        warnings.warn(f"{param_name} is deprecated for {obj.__name__} and will be removed in future versions. {msg}", category=FutureWarning, stacklevel=3)

    def decorator(obj):
        @functools.wraps(obj)
        def wrapper(*args, **kwargs):
            if param_name in kwargs:
                _warn(obj)
            return obj(*args, **kwargs)

        return wrapper

    return decorator
