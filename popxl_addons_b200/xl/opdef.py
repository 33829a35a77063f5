"""Operator registry of the graph substrate.

An `OpDef` bundles, for one operator: a reference implementation in plain torch (used for shape inference on meta
tensors, for the CPU backend and as the numerical oracle of the CUDA kernels), optional native implementations keyed
by device type (hand-written sm_100a kernels), and a vjp rule that emits the backward ops into the gradient graph.
"""
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from . import core
from .core import Op, Tensor, gcg
from .dtypes import dtype as _dtype

OPS: Dict[str, "OpDef"] = {}

# Ops that ran their torch reference on a CUDA session although a device kernel is registered for them (the kernel
# refused the operands), by op name. `STRICT[0] = True` turns such a fallback of a hot op into an error, so that a
# regression which sends e.g. the GEMMs to the library is noticed at once (the benchmark and the GPU tests switch it on).
FALLBACKS: Dict[str, int] = {}
STRICT = [False]
_HOT_PREFIXES = ("matmul", "linear_bias_act", "attention", "cross_entropy", "ce_", "layer_norm", "rms_norm", "gelu",
                 "swiglu", "gather", "adam", "rts_adam")


class NativeFallback(RuntimeError):
    """A hot op ran (or was about to run) its library / eager implementation on a GPU while strict mode is on."""


def note_fallback(name: str, detail: str = "") -> None:
    FALLBACKS[name] = FALLBACKS.get(name, 0) + 1
    if STRICT[0] and name.startswith(_HOT_PREFIXES):
        raise NativeFallback(f"op `{name}` fell back to its torch implementation on a CUDA session"
                             + (f" ({detail})" if detail else "")
                             + "; its device kernel refused the operands (dtype, alignment or layout)")


class OpDef:
    def __init__(self, name: str, impl: Optional[Callable] = None, vjp: Optional[Callable] = None,
                 infer: Optional[Callable] = None, special: Optional[Callable] = None, collective: bool = False,
                 keeps_meta: bool = False, inplace: bool = False, flops: Optional[Callable] = None):
        self.name = name
        self.impl = impl
        self.vjp = vjp
        self.infer = infer
        self.special = special  # special(executor, op, env) -> None ; handles the op entirely
        self.collective = collective
        self.keeps_meta = keeps_meta
        self.inplace = inplace
        self.flops = flops
        self.native: Dict[str, Callable] = {}
        OPS[name] = self

    def __repr__(self):
        return f"OpDef({self.name})"


def register(name: str, **kw):
    """Decorator: `@register("add", vjp=...)` on the torch reference implementation."""

    def deco(fn):
        OpDef(name, impl=fn, **kw)
        return fn

    return deco


def native(name: str, device_type: str = "cuda"):
    """Decorator that attaches a device kernel to an existing op."""

    def deco(fn):
        OPS[name].native[device_type] = fn
        return fn

    return deco


def _meta_of(t: Tensor) -> torch.Tensor:
    return torch.empty(t.shape, dtype=t.dtype.as_torch(), device="meta")


def emit(name: str, inputs: Sequence[Tensor], attrs: Optional[Dict[str, Any]] = None,
         out_names: Optional[Sequence[str]] = None, out_specs=None) -> List[Tensor]:
    """Record one op in the current graph and return its (symbolic) outputs."""
    opdef = OPS[name]
    attrs = dict(attrs or {})
    g = gcg()
    for t in inputs:
        if not isinstance(t, Tensor):
            raise TypeError(f"Not a tensor: {t!r} (input of op `{name}`)")
        if t.graph is not g:
            raise ValueError(
                f"{t} is not in the current graph {g.name}. A tensor of another graph must be passed in as a graph "
                f"input (see route_tensor_into_graph).")
    op = Op(opdef, inputs, attrs, g)
    if out_specs is None:
        if opdef.infer is not None:
            out_specs = opdef.infer(op)
        else:
            res = opdef.impl(*[_meta_of(t) for t in inputs], **attrs)
            if isinstance(res, torch.Tensor):
                res = (res,)
            out_specs = [(tuple(r.shape), _dtype.as_dtype(r.dtype), ()) for r in (res or ())]
    for i, spec in enumerate(out_specs):
        shape, dt, meta = (tuple(spec) + ((),))[:3] if not isinstance(spec, core.TensorSpec) else (
            spec.shape, spec.dtype, spec.meta_shape)
        if (not meta and opdef.keeps_meta and inputs and inputs[0].meta_shape
                and tuple(shape) == tuple(inputs[0].shape)):
            meta = inputs[0].meta_shape
        oname = out_names[i] if out_names and i < len(out_names) else name
        op.outputs.append(Tensor(g, shape, dt, oname, meta, producer=op))
    g.ops.append(op)
    g._op_created(op)
    return op.outputs


def emit1(name: str, inputs: Sequence[Tensor], attrs: Optional[Dict[str, Any]] = None, out_name=None) -> Tensor:
    return emit(name, inputs, attrs, [out_name] if out_name else None)[0]
