"""`xl.transforms`: graph-to-graph transforms of the substrate (autodiff, exchange-merging annotations)."""
import contextlib

from .autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo, autodiff  # noqa: F401  (the function shadows the submodule, as in popxl)


@contextlib.contextmanager
def merge_exchange():
    """Loads/stores issued inside are independent and may be batched on the IO stream (annotation only)."""
    yield


@contextlib.contextmanager
def io_tile_exchange():
    """`merge_exchange()` + `io_tiles()`."""
    from ..core import io_tiles

    with io_tiles():
        yield


def decompose_sum(graph):
    return graph
