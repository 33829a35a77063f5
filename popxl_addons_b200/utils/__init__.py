"""Small host-side helpers shared across the package.

Parity: popxl_addons/utils.py:25-121 (null_context, suffix_graph_name, timer, OrderedDict, WeightsDict,
overrides, duplicate_items).
"""
import collections
import contextlib
import logging
import re
import time
from collections.abc import MutableMapping
from typing import Iterable, List

import numpy as np

try:  # optional dependency, never required
    import wandb  # type: ignore

    _HAVE_WANDB = True
except Exception:  # pragma: no cover
    wandb = None
    _HAVE_WANDB = False

__all__ = [
    "null_context",
    "suffix_graph_name",
    "timer",
    "OrderedDict",
    "WeightsDict",
    "overrides",
    "duplicate_items",
]


@contextlib.contextmanager
def null_context():
    """A context manager that does nothing."""
    yield


_SUBGRAPH_TAG = re.compile(r"_subgraph\(\d+\)")


def suffix_graph_name(name: str, suffix: str) -> str:
    """`foo_subgraph(3)` + `grad` -> `foo_grad` (the numbered subgraph tag is dropped first)."""
    return _SUBGRAPH_TAG.sub("", name) + "_" + suffix


@contextlib.contextmanager
def timer(title=None, log_to_wandb=True):
    """Wall-clock timer for host-side phases (graph build, checkpoint IO). Logs minutes, and writes
    `<title>_mins` to the W&B run summary when a run is active."""
    start = time.perf_counter()
    logging.info("Starting %s", title or "")
    try:
        yield
    finally:
        mins = (time.perf_counter() - start) / 60.0
        logging.info("%s: %.2f mins", f"{title} duration" if title else "Duration", mins)
        if log_to_wandb and title and _HAVE_WANDB and wandb.run is not None:
            wandb.run.summary[title.lower().replace(" ", "_") + "_mins"] = mins


class OrderedDict(collections.OrderedDict):
    """Ordered dict with positional access (`idx`) and a line-per-item repr."""

    def idx(self, idx: int):
        for n, v in enumerate(self.values()):
            if n == idx:
                return v
        if idx < 0:
            return list(self.values())[idx]
        raise IndexError(idx)

    def __repr__(self):
        body = "".join(f"{k}: {v},\n" for k, v in self.items())
        return "{\n" + body + "}" if body else "{}"


class WeightsDict(MutableMapping):
    """Mapping variable -> host array that refuses entries whose dtype or host shape disagree with the variable."""

    def __init__(self, *args, **kwargs):
        self._items = {}
        if args or kwargs:
            self.update(*args, **kwargs)

    def __setitem__(self, var, array):
        from ..xl.dtypes import dtype as _dtype

        array_dtype = _dtype.as_dtype(array.dtype)
        try:
            var.dtype.as_numpy()
            host_float32_ok = False
        except TypeError:  # bf16 / fp8 variables take float32 host data
            host_float32_ok = array.dtype == np.float32
        if var.dtype != array_dtype and not host_float32_ok:
            raise ValueError(f"{var}: tensor and weight dtypes do not equal {var.dtype} != {array_dtype}")
        if tuple(var.shape_on_host) != tuple(array.shape):
            raise ValueError(f"{var}: tensor and weight shapes do not equal {var.shape_on_host} != {array.shape}")
        self._items[var] = array

    def __getitem__(self, var):
        return self._items[var]

    def __delitem__(self, var):
        del self._items[var]

    def __len__(self):
        return len(self._items)

    def __iter__(self):
        return iter(self._items)


def overrides(cls, base_cls, method: str) -> bool:
    """True when `cls` provides its own implementation of `method` rather than inheriting `base_cls`'s."""
    return getattr(cls, method) is not getattr(base_cls, method)


def duplicate_items(iterable: Iterable) -> List:
    """Items seen more than once, in first-seen order: [7,5,5,1,2,7] -> [7,5]."""
    counts = collections.Counter(iterable)
    return [k for k, c in counts.items() if c > 1]
