"""Element types of the graph substrate: thin named wrappers that convert to/from numpy and torch dtypes.

The two 8-bit float formats keep the names the add-on API uses (`float8_143` = 1 sign, 4 exponent, 3 mantissa bits;
`float8_152` = 1-5-2) and map to the OCP e4m3fn / e5m2 encodings that Blackwell tensor cores consume.
Parity: the `popxl.dtype` surface used by popxl_addons (e.g. variable_factory.py:82-97, ops/fp8_utils.py:6-23).
"""
from typing import Any

import numpy as np
import torch

__all__ = [
    "dtype", "float64", "float32", "float16", "bfloat16", "float8_143", "float8_152",
    "int64", "int32", "int16", "int8", "uint64", "uint32", "uint16", "uint8", "bool_",
]


class dtype:
    _by_name = {}
    _by_torch = {}
    _by_numpy = {}

    def __init__(self, name, torch_dtype, numpy_dtype, is_float, is_int, is_signed, bits):
        self.name = name
        self._torch = torch_dtype
        self._numpy = None if numpy_dtype is None else np.dtype(numpy_dtype)
        self.is_floating_point = is_float
        self.is_int = is_int
        self.is_signed = is_signed
        self.bits = bits
        dtype._by_name[name] = self
        dtype._by_torch.setdefault(torch_dtype, self)
        if self._numpy is not None:
            dtype._by_numpy.setdefault(self._numpy, self)

    @property
    def itemsize(self) -> int:
        return self.bits // 8

    def as_numpy(self) -> np.dtype:
        if self._numpy is None:
            raise TypeError(f"{self.name} has no numpy equivalent")
        return self._numpy

    def as_torch(self) -> torch.dtype:
        return self._torch

    @classmethod
    def as_dtype(cls, x: Any) -> "dtype":
        """Convert a dtype-like (our dtype, torch/numpy dtype, type name, array, tensor, python scalar) to a dtype."""
        if isinstance(x, dtype):
            return x
        if isinstance(x, torch.dtype):
            return cls._by_torch[x]
        if isinstance(x, str):
            if x in cls._by_name:
                return cls._by_name[x]
            return cls._by_numpy[np.dtype(x)]
        if isinstance(x, torch.Tensor):
            return cls._by_torch[x.dtype]
        if hasattr(x, "dtype") and not isinstance(x, type):
            return cls.as_dtype(x.dtype)
        if isinstance(x, bool):
            return bool_
        if isinstance(x, int):
            return int32
        if isinstance(x, float):
            return float32
        try:
            return cls._by_numpy[np.dtype(x)]
        except Exception:
            raise TypeError(f"cannot interpret {x!r} as a dtype") from None

    def __repr__(self):
        return self.name

    def __hash__(self):
        return hash(self.name)

    def __eq__(self, other):
        return isinstance(other, dtype) and other.name == self.name


float64 = dtype("float64", torch.float64, np.float64, True, False, True, 64)
float32 = dtype("float32", torch.float32, np.float32, True, False, True, 32)
float16 = dtype("float16", torch.float16, np.float16, True, False, True, 16)
bfloat16 = dtype("bfloat16", torch.bfloat16, None, True, False, True, 16)
float8_143 = dtype("float8_143", torch.float8_e4m3fn, None, True, False, True, 8)
float8_152 = dtype("float8_152", torch.float8_e5m2, None, True, False, True, 8)
int64 = dtype("int64", torch.int64, np.int64, False, True, True, 64)
int32 = dtype("int32", torch.int32, np.int32, False, True, True, 32)
int16 = dtype("int16", torch.int16, np.int16, False, True, True, 16)
int8 = dtype("int8", torch.int8, np.int8, False, True, True, 8)
uint64 = dtype("uint64", torch.uint64, np.uint64, False, True, False, 64)
uint32 = dtype("uint32", torch.uint32, np.uint32, False, True, False, 32)
uint16 = dtype("uint16", torch.uint16, np.uint16, False, True, False, 16)
uint8 = dtype("uint8", torch.uint8, np.uint8, False, True, False, 8)
bool_ = dtype("bool", torch.bool, np.bool_, False, False, False, 8)


def to_torch(data, dt: "dtype" = None) -> torch.Tensor:
    """Host data (numpy / torch / scalar / nested list) -> CPU torch tensor of dtype `dt`."""
    if isinstance(data, torch.Tensor):
        t = data.detach()
    else:
        arr = np.asarray(data)
        if arr.dtype == np.uint16:
            t = torch.from_numpy(arr.view(np.int16).copy()).view(torch.uint16)
        elif arr.dtype == np.uint32:
            t = torch.from_numpy(arr.view(np.int32).copy()).view(torch.uint32)
        elif arr.dtype == np.uint64:
            t = torch.from_numpy(arr.view(np.int64).copy()).view(torch.uint64)
        else:
            t = torch.from_numpy(np.array(arr, order="C", copy=True))
    if dt is not None and t.dtype != dt.as_torch():
        t = t.to(dt.as_torch())
    return t


def to_numpy(t: torch.Tensor) -> np.ndarray:
    """Torch tensor (any device) -> numpy; bf16 / fp8 come back as float32 because numpy cannot hold them."""
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
        t = t.float()
    if t.dtype == torch.uint16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    if t.dtype == torch.uint64:
        return t.view(torch.int64).numpy().view(np.uint64)
    return t.numpy()
