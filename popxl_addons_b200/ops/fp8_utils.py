"""Parameters of the two 8-bit float formats.

`float8_143` / `float8_152` here are the OCP e4m3fn / e5m2 encodings Blackwell tensor cores consume (max 448 /
57344), not the Graphcore encodings of the same names (exponent bias 8 / 16, max 240 / 57344:
popxl_addons/ops/fp8_utils.py:6-23). Scale selection only depends on the format's maximum and mantissa width, which
are parameters of every routine below.
"""
from collections import namedtuple

from .. import xl

__all__ = ["fp8_format", "FP8_FORMATS", "FpDef", "ieee_fp32_no_denorms", "ieee_fp16_denorms", "float8_152_def",
           "float8_143_def"]

# Format descriptions under the reference's names and field order. The two 8-bit entries describe the encodings this
# package computes with (see above), so their bias / maximum differ from the reference's table.
FpDef = namedtuple("FpDef", ["num_exp_bits", "num_mantissa_bits", "fix_exponent_bias", "include_denorm", "has_nans",
                             "max_value", "max_exp", "min_exp"])
ieee_fp32_no_denorms = FpDef(8, 23, 127, False, True, 3.4028235e38, 127, -126)
ieee_fp16_denorms = FpDef(5, 10, 15, True, True, 65504, 15, -14)
float8_152_def = FpDef(5, 2, 15, True, True, 57344, 15, -16)   # e5m2: IEEE-like, smallest subnormal 2^-16
float8_143_def = FpDef(4, 3, 7, True, False, 448, 8, -9)       # e4m3fn: one NaN code only, smallest subnormal 2^-9

FP8_FORMATS = {
    "float8_143": dict(max=448.0, mantissa_bits=3, exponent_bits=4, exponent_bias=7, min_normal_exp=-6),
    "float8_152": dict(max=57344.0, mantissa_bits=2, exponent_bits=5, exponent_bias=15, min_normal_exp=-14),
}


def fp8_format(dtype: xl.dtype) -> dict:
    if dtype.name not in FP8_FORMATS:
        raise ValueError(f"dtype must be float8_143 or float8_152, got {dtype}")
    return FP8_FORMATS[dtype.name]
