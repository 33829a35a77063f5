"""`xl.ops.negative_log_likelihood` (popxl/ops/negative_log_likelihood.py)."""
try:
    from typing import Literal
except ImportError:  # pragma: no cover
    from typing_extensions import Literal

from . import nll_loss, nll_loss_with_softmax_grad  # noqa: F401

REDUCTION_TYPE = Literal["mean", "sum", "none"]

__all__ = ["nll_loss", "nll_loss_with_softmax_grad", "REDUCTION_TYPE"]
