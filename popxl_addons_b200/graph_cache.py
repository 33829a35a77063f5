"""Re-use of graphs created from the same function and argument specs.

Parity: popxl_addons/graph_cache.py:14-118.
"""
import inspect
import weakref
from functools import wraps
from typing import Any, Callable, Dict, Mapping

from . import xl
from .xl import ops

__all__ = ["GraphCache", "function", "get_function_hash", "argument_hash", "tensor_hash", "bound_arguments"]


def tensor_hash(t) -> int:
    """Tensors are interchangeable for caching when shape, dtype and meta-shape agree."""
    return hash((tuple(t.shape), t.dtype, tuple(t.meta_shape or ())))


def argument_hash(arg: Any) -> int:
    from .graph import BoundGraph, GraphWithNamedArgs

    if isinstance(arg, (xl.Tensor, xl.TensorSpec)):
        return tensor_hash(arg)
    if isinstance(arg, BoundGraph):
        return hash((id(arg.graph), tuple(sorted((a.uid, b.uid) for a, b in arg.args.items()))))
    if isinstance(arg, GraphWithNamedArgs):
        return hash(id(arg.graph))
    if isinstance(arg, Mapping):
        return hash(tuple((argument_hash(k), argument_hash(v)) for k, v in arg.items()))
    if isinstance(arg, (list, tuple)):
        return hash(tuple(argument_hash(a) for a in arg))
    try:
        return hash(arg)
    except TypeError:
        return id(arg)


def bound_arguments(fn: Callable, *args, **kwargs) -> Dict[str, Any]:
    target = fn.build if hasattr(fn, "build") and not inspect.isroutine(fn) else fn
    bound = inspect.signature(target).bind(*args, **kwargs)
    bound.apply_defaults()
    return dict(bound.arguments)


def get_function_hash(fn: Callable, *args, **kwargs) -> int:
    """Hash of (function identity, placement context, hash of every bound argument)."""
    from .xl.core import current_device, current_tile_set

    # the callable's own hash: two module instances that define equal `__hash__` (same configuration) share graphs
    try:
        fn_hash = hash(fn)
    except TypeError:
        fn_hash = id(fn)
    parts = [fn_hash, current_device(), current_tile_set()]
    for name, value in bound_arguments(fn, *args, **kwargs).items():
        parts.append((name, argument_hash(value)))
    return hash(tuple(parts))


class GraphCache:
    """Per-Ir cache `hash -> Graph`. Irs are held weakly so a cache never keeps an Ir alive."""

    def __init__(self):
        self._per_ir: "weakref.WeakKeyDictionary[xl.Ir, Dict[int, xl.Graph]]" = weakref.WeakKeyDictionary()

    def create_graph(self, fn: Callable, *args, **kwargs) -> xl.Graph:
        ir = xl.gcg().ir
        table = self._per_ir.setdefault(ir, {})
        key = get_function_hash(fn, *args, **kwargs)
        if key not in table:
            table[key] = ir.create_graph(fn, *args, **kwargs)
        return table[key]


_FUNCTION_CACHE = GraphCache()


def function(fn: Callable) -> Callable:
    """Decorator: calls of `fn` are outlined. One graph is created per distinct argument signature and every call
    becomes an `ops.call` of it. Non-tensor arguments are baked into the graph (and into the cache key)."""

    @wraps(fn)
    def wrapper(*args, **kwargs):
        graph = _FUNCTION_CACHE.create_graph(fn, *args, **kwargs)
        tensors = []
        for value in bound_arguments(fn, *args, **kwargs).values():
            if isinstance(value, xl.Tensor):
                tensors.append(value)
            elif isinstance(value, (list, tuple)) and value and all(isinstance(v, xl.Tensor) for v in value):
                tensors.extend(value)
        outs = ops.call(graph, *tensors)
        if len(outs) == 0:
            return None
        if len(outs) == 1:
            return outs[0]
        return outs

    return wrapper
