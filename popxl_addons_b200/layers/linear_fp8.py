"""Linear layer whose matmuls run on FP8 tensor cores, forward (e4m3) and backward (e5m2 gradients).

Forward: power-of-two scales for `x` and `w` (from amax, from an MSE search, or fixed), cast both to float8_143,
`matmul_pow2scaled` un-scales the fp32 accumulator; the FP8 operands and scales are kept in `aux` for the hand-written
backward pass, which casts `dL/dy` to float8_152 and runs the two gradient GEMMs in FP8 as well.
Parity: popxl_addons/layers/linear_fp8.py:18-131.
"""
from functools import partial
from typing import Optional

import numpy as np

from .. import xl
from ..module import Module
from ..ops.fp8_amax_scale import fp8_amax_scale
from ..ops.fp8_mse_scale import fp8_mse_scale
from ..xl import ops
from .linear import truncnorm_init

__all__ = ["LinearFP8"]


class LinearFP8(Module):
    def __init__(self, out_features: int, bias: bool = True, scale_metric: str = "amax", scale: int = 0,
                 replica_grouping: Optional[xl.ReplicaGrouping] = None):
        super().__init__()
        if scale_metric not in ("amax", "mse", "manual_scale"):
            raise ValueError(f"scale_metric must be one of amax, mse, manual_scale. Not: {scale_metric}")
        self.out_features = out_features
        self.bias = bias
        self.scale_metric = scale_metric
        self.scale = scale
        self.replica_grouping = replica_grouping

    def _scale(self, t: xl.Tensor, dtype: xl.dtype) -> xl.Tensor:
        if self.scale_metric == "amax":
            return fp8_amax_scale(t, dtype)
        if self.scale_metric == "mse":
            return fp8_mse_scale(t, dtype)
        return xl.constant(self.scale, xl.int32, "fp8_scale")

    def build(self, x: xl.Tensor) -> xl.Tensor:
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w = self.add_variable_input("weight", partial(truncnorm_init, (x.shape[-1], self.out_features), 0.02, np_dt),
                                    x.dtype, replica_grouping=self.replica_grouping)
        sw, sx = self._scale(w, xl.float8_143), self._scale(x, xl.float8_143)
        w8 = ops.pow2scale_cast_to_fp8(w, sw, xl.float8_143)
        x8 = ops.pow2scale_cast_to_fp8(x, sx, xl.float8_143)
        out_dt = xl.float16 if x.dtype == xl.float32 else x.dtype
        y = ops.matmul_pow2scaled(x8, w8, ops.negate(ops.add(sw, sx)), out_dt)
        if y.dtype != x.dtype:
            y = ops.cast(y, x.dtype)
        if self.bias:
            b = self.add_variable_input("bias", partial(np.zeros, (self.out_features,), np_dt), x.dtype,
                                        replica_grouping=self.replica_grouping)
            y = y + b
        self.aux["w_fp8"], self.aux["x_fp8"] = w8, x8
        self.aux["w_scale"], self.aux["x_scale"] = sw, sx
        self.aux["dtype"] = x.dtype
        self.aux["has_bias"] = self.bias
        return y

    def build_grad(self, dLdy: xl.Tensor):
        w8, x8 = self.aux["w_fp8"], self.aux["x_fp8"]
        sw, sx = self.aux["w_scale"], self.aux["x_scale"]
        dt = self.aux["dtype"]
        out_dt = xl.float16 if dt == xl.float32 else dt
        # gradients use the wide-exponent format; leave 3 octaves of headroom for accumulation growth
        sg = ops.clip(ops.sub(ops.cast(fp8_amax_scale(dLdy, xl.float8_152), xl.float32), 3.0), -31.0, 31.0)
        sg = ops.cast(sg, xl.int32)
        g8 = ops.pow2scale_cast_to_fp8(dLdy, sg, xl.float8_152)
        dLdx = ops.matmul_pow2scaled(g8, ops.transpose(w8), ops.negate(ops.add(sg, sw)), out_dt)
        dLdw = ops.transpose(ops.matmul_pow2scaled(ops.transpose(g8), x8, ops.negate(ops.add(sg, sx)), out_dt))
        if dLdx.dtype != dt:
            dLdx, dLdw = ops.cast(dLdx, dt), ops.cast(dLdw, dt)
        self.var_grad["weight"] = dLdw
        if self.aux["has_bias"]:
            self.var_grad["bias"] = ops.sum(dLdy, axis=0)
        return dLdx

    @staticmethod
    def torch_mapping(variables, nn_layer, dtype: xl.dtype = xl.float32):
        """Host data for `variables` from a `torch.nn.Linear` (whose weight is `(out, in)`), converted to `dtype`."""
        from ..utils import WeightsDict
        from ..xl.utils import to_numpy

        out = {variables.weight: np.ascontiguousarray(to_numpy(nn_layer.weight.data, dtype).T)}
        if "bias" in variables.keys():
            out[variables.bias] = to_numpy(nn_layer.bias.data, dtype)
        return WeightsDict(out)
