"""Cross-entropy on logits, plain and with the gradient fused into the forward computation.

Parity: popxl_addons/ops/cross_entropy.py:10-66.
"""
from typing import Optional, Tuple, Union

from .. import xl
from ..xl import ops

__all__ = ["cross_entropy", "cross_entropy_with_grad"]


def cross_entropy(x: xl.Tensor, labels: xl.Tensor, ignore_index: Optional[int] = None,
                  reduction: str = "mean") -> xl.Tensor:
    """`nll(softmax(x), labels)`; differentiable through autodiff."""
    return ops.nll_loss(ops.softmax(x, axis=-1), labels, ignore_index=ignore_index, reduction=reduction)


def cross_entropy_with_grad(x: xl.Tensor, labels: xl.Tensor, loss_scaling: Union[float, xl.Tensor] = 1,
                            ignore_index: Optional[int] = None,
                            reduction: str = "mean") -> Tuple[xl.Tensor, xl.Tensor]:
    """Loss and d(loss * loss_scaling)/dx in one pass (no separate backward graph needed for the loss)."""
    if not isinstance(loss_scaling, xl.Tensor):
        loss_scaling = xl.constant(loss_scaling, xl.float32, "loss_scaling")
    return ops.cross_entropy_with_grad(x, labels, loss_grad=loss_scaling, reduction=reduction,
                                       ignore_index=ignore_index)
