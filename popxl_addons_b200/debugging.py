"""Device-side prints gated by the environment variable `MODEL_LOG_LEVEL` (TRACE < DEBUG < INFO < WARN).
Parity: popxl_addons/debugging.py:14-45."""
import os
from typing import Optional

from . import xl
from .xl import ops

__all__ = ["print_tensor", "print_text"]

_LEVELS = {"TRACE": 0, "DEBUG": 1, "INFO": 2, "WARN": 3, "OFF": 4}


def _enabled(level: str) -> bool:
    if level not in _LEVELS:
        raise ValueError(f"level must be one of {list(_LEVELS)}. Not: {level}")
    current = os.environ.get("MODEL_LOG_LEVEL", "OFF").upper()
    return _LEVELS.get(current, 4) <= _LEVELS[level]


def print_tensor(t: xl.Tensor, *args, level: str = "DEBUG", **kwargs) -> xl.Tensor:
    """`ops.print_tensor` when the log level allows it, else `t` unchanged."""
    return ops.print_tensor(t, *args, **kwargs) if _enabled(level) else t


def print_text(text: str, num: Optional[xl.Tensor] = None, level: str = "DEBUG"):
    """Print `text` at run time (a tensor is needed to anchor the print; a dummy constant is used if none given)."""
    if not _enabled(level):
        return num
    anchor = num if num is not None else xl.constant(0, xl.int32)
    return ops.print_tensor(anchor, title=text)
