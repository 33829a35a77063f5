"""Ordered, named groups of host streams.

Parity: popxl_addons/streams.py:12-69.
"""
from typing import Iterable, Mapping, Tuple, Union

from . import xl
from .utils import OrderedDict

__all__ = ["InputStreams", "OutputStreams"]


class _Streams:
    _factory = None

    def __init__(self, **specs: Tuple[Iterable[int], xl.dtype]):
        self._streams = OrderedDict()
        for name, (shape, dt) in specs.items():
            self._streams[name] = type(self)._factory(shape, dt, name)

    @classmethod
    def from_streams(cls, streams: Union[Iterable, Mapping[str, object]]):
        """From existing streams: an iterable of streams (named by their `tensor_id`, as in the reference) or a mapping
        name -> stream."""
        self = cls()
        if isinstance(streams, Mapping):
            for name, s in streams.items():
                self._streams[name] = s
        else:
            for s in streams:
                self._streams[s.tensor_id] = s
        return self

    def __contains__(self, name) -> bool:
        return name in self._streams

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        try:
            return self._streams[name]
        except KeyError:
            raise AttributeError(f"No stream named '{name}'. Available: {list(self._streams)}") from None

    def __getitem__(self, key: Union[int, slice, str]):
        if isinstance(key, str):
            return self._streams[key]
        return list(self._streams.values())[key]

    def __iter__(self):
        return iter(self._streams.values())

    def __len__(self):
        return len(self._streams)

    def keys(self):
        return self._streams.keys()

    def values(self):
        return self._streams.values()

    def items(self):
        return self._streams.items()

    def __repr__(self):
        return f"{type(self).__name__}({dict(self._streams)})"


class InputStreams(_Streams):
    _factory = staticmethod(xl.h2d_stream)


class OutputStreams(_Streams):
    _factory = staticmethod(xl.d2h_stream)
