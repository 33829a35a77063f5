"""Differentiable all-reduce for tensor parallelism with the two autograd pairings.

* `identical_inputs`      — forward identity, backward all-reduce (Megatron's *f*).
* `identical_grad_inputs` — forward all-reduce, backward identity (Megatron's *g*).

In the tensor-parallel `Linear` layers of this package the *g* all-reduce is fused into the row-parallel GEMM's
epilogue (GEMM -> reduce over NVLink) instead of running as a separate op.
Parity: popxl_addons/ops/replicated_all_reduce_TP/replicated_all_reduce_TP.py:24-122.
"""
from typing import Optional

from .. import xl
from ..xl.ops import collectives as _c

__all__ = ["replicated_all_reduce", "replicated_all_reduce_identical_inputs",
           "replicated_all_reduce_identical_grad_inputs"]


def _check(op):
    name = _c._norm_op(op)
    if name != "add":
        raise ValueError("The tensor-parallel all-reduce supports `add` only")
    return name


def replicated_all_reduce(t: xl.Tensor, op="add", group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    return _c.replicated_all_reduce(t, _check(op), group)


def replicated_all_reduce_identical_inputs(t: xl.Tensor, op="add",
                                           group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    return _c.replicated_all_reduce(t, _check(op), group, identical_inputs=True)


def replicated_all_reduce_identical_grad_inputs(t: xl.Tensor, op="add",
                                                group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    return _c.replicated_all_reduce(t, _check(op), group, identical_grad_inputs=True)


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
