"""`xl.ops.utils` (popxl/ops/utils.py): argument checks shared by op wrappers."""
from typing import Optional

from ..core import Tensor, gcg

__all__ = ["check_in_graph", "check_tensor_ipu_and_tile_set", "convert_optional_float", "convert_optional_int"]


def check_in_graph(graph, **tensors: Tensor) -> None:
    """Raise if a tensor does not belong to `graph`."""
    for name, t in tensors.items():
        if not isinstance(t, Tensor):
            raise TypeError(f"Not a tensor: {name} = {t!r}")
        if t.graph is not graph:
            raise ValueError(f"{name} is not in the graph {graph.name}: {t}")


def check_tensor_ipu_and_tile_set(**tensors: Tensor) -> None:
    """Raise if the tensors were placed on different device slots."""
    placed = {}
    for name, t in tensors.items():
        dev = getattr(getattr(t, "producer", None), "device_index", None)
        if dev is not None:
            placed[name] = dev
    if len(set(placed.values())) > 1:
        raise ValueError(f"The input tensors are located on different IPUs: {placed}")


def convert_optional_float(name: str, value: Optional[float]):
    if value is None:
        return None
    try:
        return float(value)
    except (TypeError, ValueError):
        raise TypeError(f"{name} must be a float or None, got {value!r}") from None


def convert_optional_int(name: str, value: Optional[int]):
    if value is None:
        return None
    if int(value) != value:
        raise TypeError(f"{name} must be an int or None, got {value!r}")
    return int(value)
