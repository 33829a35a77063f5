"""`linear_layout`: value-identity copy into a plain row-major contiguous tensor.

The reference op exists to force a linear tile mapping on the IPU; on a GPU the only layout question is contiguity,
so this returns a contiguous copy (grain size `bs` is accepted and ignored).
Parity: popxl_addons/ops/linear_layout/linear_layout.py:20-47.
"""
import torch

from .. import xl
from ..xl.opdef import OpDef, emit1

__all__ = ["linear_layout"]

OpDef("linear_layout", impl=lambda t, bs: t.contiguous().clone() if t.device.type != "meta" else torch.empty_like(t),
      vjp=lambda ctx, op, gs: [gs[0]])


def linear_layout(t: xl.Tensor, bs: int = 1) -> xl.Tensor:
    return emit1("linear_layout", [t], {"bs": int(bs)})


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
