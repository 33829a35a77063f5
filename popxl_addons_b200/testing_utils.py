"""Helpers for tests: count ops, and build-and-run a module in one call.
Parity: popxl_addons/testing_utils.py:15-107."""
from typing import Callable, Iterable, Optional, Tuple, Union

import numpy as np

from . import xl
from .module import Module
from .xl import ops

__all__ = ["ops_of_type", "TensorInput", "run_module"]


def ops_of_type(ops: Iterable, op_type: Union[str, type]) -> int:
    """Number of ops of type `op_type`: an op name of this package (`"matmul"`), a popart-style type name (`"MatMul"`,
    `"Accumulate"`) or a class whose name is one of those with an `Op` suffix. `ops` may be a graph's `ops` or the
    popart-style views `graph._pb_graph.getOps()` returns."""
    from .xl.core import pb_op_type

    name = op_type if isinstance(op_type, str) else getattr(op_type, "__name__", str(op_type))
    names = {name, name[:-2] if name.endswith("Op") else name}
    count = 0
    for o in ops:
        o = getattr(o, "_op", o)
        if o.opdef.name in names or pb_op_type(o) in names:
            count += 1
    return count


class TensorInput:
    """Marks a positional argument of `run_module` as host data to be streamed in as a tensor."""

    def __init__(self, data: np.ndarray, dtype: Optional[xl.dtype] = None):
        self.data = np.asarray(data)
        self.dtype = dtype or xl.dtype.as_dtype(np.float32 if self.data.dtype == np.float64 else self.data.dtype)


def run_module(module: Module, *args, weights: Optional[Callable] = None, device: str = "auto",
               **kwargs) -> Tuple[np.ndarray, ...]:
    """Build `module` with the given arguments (`TensorInput`s become host-loaded tensors, everything else is passed
    through), initialise its variables (optionally overwritten by `weights(variables) -> {var: array}`), run one
    step and return the outputs as numpy arrays."""
    ir = xl.Ir()
    feeds = {}
    with ir.main_graph:
        def convert(a):
            if isinstance(a, TensorInput):
                stream = xl.h2d_stream(a.data.shape, a.dtype)
                feeds[stream] = a.data
                return ops.host_load(stream)
            return a

        targs = [convert(a) for a in args]
        tkwargs = {k: convert(v) for k, v in kwargs.items()}
        factories, graph = module.create_graph(*targs, **tkwargs)
        variables = factories.init()
        tensor_args = [a for a in targs if isinstance(a, xl.Tensor)]
        outs = graph.bind(variables).call(*tensor_args)
        streams = [xl.d2h_stream(o.shape, o.dtype) for o in outs]
        for s, o in zip(streams, outs):
            ops.host_store(s, o)
    session = xl.Session(ir, device)
    if weights is not None:
        session.write_variables_data(weights(variables))
    with session:
        results = session.run(feeds)
    return tuple(results[s] for s in streams)
