"""Parameters of the two 8-bit float formats.

`float8_143` / `float8_152` here are the OCP e4m3fn / e5m2 encodings Blackwell tensor cores consume (max 448 /
57344), not the Graphcore encodings of the same names (exponent bias 8 / 16, max 240 / 57344:
popxl_addons/ops/fp8_utils.py:6-23). Scale selection only depends on the format's maximum and mantissa width, which
are parameters of every routine below.
"""
from .. import xl

__all__ = ["fp8_format", "FP8_FORMATS"]

FP8_FORMATS = {
    "float8_143": dict(max=448.0, mantissa_bits=3, exponent_bits=4, exponent_bias=7, min_normal_exp=-6),
    "float8_152": dict(max=57344.0, mantissa_bits=2, exponent_bits=5, exponent_bias=15, min_normal_exp=-14),
}


def fp8_format(dtype: xl.dtype) -> dict:
    if dtype.name not in FP8_FORMATS:
        raise ValueError(f"dtype must be float8_143 or float8_152, got {dtype}")
    return FP8_FORMATS[dtype.name]
