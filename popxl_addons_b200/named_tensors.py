"""Named collections of tensors (and of their host data).

Parity: popxl_addons/named_tensors.py:16-47.
"""
from typing import Dict, Mapping, Tuple

import numpy as np

from .dot_tree import DotTree
from . import xl

__all__ = ["NamedTensors", "NamedTensorData", "print_named_tensors"]


class NamedTensorData(DotTree):
    """DotTree of numpy arrays."""


class NamedTensors(DotTree):
    """DotTree whose leaves are tensors."""

    @property
    def tensors(self) -> Tuple[xl.Tensor, ...]:
        """All leaves, ordered by tensor name (so the order is independent of insertion order)."""
        return tuple(sorted(self.to_dict().values(), key=lambda t: t.name))

    @property
    def named_tensors(self) -> Dict[str, xl.Tensor]:
        return self.to_dict()

    def remap(self, mapping: Mapping[xl.Tensor, xl.Tensor]) -> "NamedTensors":
        """Copy in which every tensor that is a key of `mapping` is replaced by the mapped tensor."""
        return self.from_dict({k: mapping.get(t, t) for k, t in self.to_dict().items()})


def print_named_tensors(named_tensors: NamedTensors) -> NamedTensors:
    """Emit a device-side print for every tensor; returns the (passed-through) tensors under the same names."""
    from .xl import ops

    return NamedTensors.from_dict({k: ops.print_tensor(t, k) for k, t in named_tensors.to_dict().items()})
