"""`xl.ops.conv` (popxl/ops/conv.py): convolution and the names of its padding modes."""
try:
    from typing import Literal
except ImportError:  # pragma: no cover
    from typing_extensions import Literal

from . import conv  # noqa: F401

PadType = Literal["not_set", "same_upper", "same_lower", "valid"]

__all__ = ["conv", "PadType"]
