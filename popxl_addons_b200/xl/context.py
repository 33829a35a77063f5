"""`xl.context`: the build context under popxl's module path (popxl/context.py): current graph, device slot and tile
set, and the decorators popxl puts on op wrappers (they attach source locations for the Graphcore profiler; here they
return the function unchanged)."""
import contextlib
import functools

from .core import (current_device, current_tile_set, gcg, get_current_graph, gir, gmg, in_sequence, io_tiles, ipu,  # noqa: F401
                   name_scope)

__all__ = ["get_current_context", "get_current_graph", "get_main_graph", "gcg", "gmg", "gir", "op_debug_context",
           "debug_context_frame_offset", "name_scope", "in_sequence", "ipu", "io_tiles"]

get_main_graph = gmg


class Context:
    """View of the build state of the current thread."""

    @property
    def graph(self):
        return gcg()

    @property
    def ipu_id(self) -> int:
        return current_device()

    @property
    def io_tile_set(self) -> str:
        return current_tile_set()

    @property
    def in_sequence(self):
        from .core import _STATE

        return _STATE.sequence[-1] if _STATE.sequence else None

    def register_op_created_hook(self, fn):
        return gcg().register_op_created_hook(fn)

    def remove_op_created_hook(self, handle):
        return gcg().remove_op_created_hook(handle)


_CONTEXT = Context()


def get_current_context() -> Context:
    return _CONTEXT


def op_debug_context(arg):
    """`@op_debug_context` or `@op_debug_context("name")` on an op wrapper."""
    if callable(arg):
        return arg
    return lambda fn: fn


def debug_context_frame_offset(offset: int):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            return fn(*a, **k)

        return wrapper

    return deco


@contextlib.contextmanager
def _execution_context(_kind=None):
    """popxl places ops into program fragments (weights-from-host, weights-to-host, ...); every op of this substrate runs
    in the main program, variables are read and written by the session directly."""
    yield
