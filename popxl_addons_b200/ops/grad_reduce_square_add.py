"""Sum of squares of a loss-scaled gradient, un-scaled: `sum((t / loss_scaling)^2)` as one fp32 scalar.

Used for global-norm clipping. In the fused reduce-scatter + Adam path the same partial sums are produced while the
reduced shard is still in registers; this standalone op is a single-pass block-reduction kernel on CUDA.
Parity: popxl_addons/ops/grad_reduce_square_add/grad_reduce_square_add.py:19-57.
"""
from typing import Union

import torch

from .. import xl
from ..xl.opdef import OpDef, emit1

__all__ = ["grad_reduce_square_add"]


def _impl(t, scale):
    if t.device.type == "meta":
        return torch.empty((), dtype=torch.float32, device="meta")
    tf = t.float()
    return (tf * tf).sum() * scale.float().reshape(())


OpDef("grad_reduce_square_add", impl=_impl)


def grad_reduce_square_add(t: xl.Tensor, loss_scaling: Union[int, float, xl.Tensor]) -> xl.Tensor:
    if isinstance(loss_scaling, xl.Tensor):
        ls = xl.ops.cast(loss_scaling, xl.float32)
        scale = xl.ops.div(xl.constant(1.0, xl.float32), xl.ops.mul(ls, ls))
    else:
        scale = xl.constant(1.0 / (float(loss_scaling) * float(loss_scaling)), xl.float32)
    return emit1("grad_reduce_square_add", [t, scale], out_name="grad_reduced")


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
