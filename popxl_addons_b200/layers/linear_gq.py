"""Inference-only Linear with 4-bit group-quantised weights; the dequantisation is fused into the GEMM on CUDA.

`dim` selects the axis the quantisation groups run along: `-1`/`1` the output features, `0` the input features
(the usual "groups of 64 along the input dimension"). Variables: `weight_compressed` uint16 `(U, C/gs, gs/4)`,
`weight_decompression_scale` / `_bias` `(U, C/gs, 1)`, where `C` is the grouped axis and `U` the other one.
Parity: popxl_addons/layers/linear_gq.py:19-136.
"""
from functools import partial
from typing import Optional

import numpy as np

from .. import xl
from ..utils import WeightsDict
from ..xl.utils import to_numpy
from ..module import Module
from ..named_tensors import NamedTensors
from ..ops.group_quantize_decompress import group_quantize_compress_numpy
from ..xl.opdef import OpDef, emit1

__all__ = ["LinearGQ", "linear_gq_window", "linear_gq_window_t", "interleave_scale_zero"]

import torch  # noqa: E402

from ..ops.group_quantize_decompress import _decompress_ref  # noqa: E402


def _linear_gq_ref(x, packed, scale, bias, *b, dim):
    if x.device.type == "meta":
        u, g, w = packed.shape
        n = g * w * 4 if dim in (-1, 1) else u
        return torch.empty((*x.shape[:-1], n), dtype=x.dtype, device="meta")
    w = _decompress_ref(packed, scale, bias)
    if dim not in (-1, 1):
        w = w.t()
    y = torch.matmul(x, w.to(x.dtype))
    if b:
        y = y + b[0].to(y.dtype)
    return y


OpDef("linear_gq", impl=_linear_gq_ref,
      flops=lambda op: 2 * op.inputs[0].shape[-1] * op.outputs[0].nelms)


def _linear_gq_window_ref(x, packed, scale, bias, *b, x_col, k, act_from_col):
    if x.device.type == "meta":
        return torch.empty((x.shape[0], packed.shape[0]), dtype=x.dtype, device="meta")
    w = _decompress_ref(packed, scale, bias)  # (out, k)
    y = torch.matmul(x[:, x_col:x_col + k], w.t().to(x.dtype))
    if b:
        y = y + b[0].to(y.dtype)
    if act_from_col is not None and act_from_col < y.shape[1]:
        y = torch.cat([y[:, :act_from_col], torch.nn.functional.gelu(y[:, act_from_col:].float()).to(y.dtype)], dim=1)
    return y


OpDef("linear_gq_window", impl=_linear_gq_window_ref,
      flops=lambda op: 2 * op.attrs["k"] * op.outputs[0].nelms)


def interleave_scale_zero(scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """`(out, groups, 1)` scale and zero point -> one `(groups, out, 2)` tensor of (scale, zero) pairs: the layout in
    which the fused small-batch kernel reads the eight output columns of an MMA tile as one 32-byte segment."""
    return torch.stack([scale.reshape(scale.shape[0], -1).t(), zero.reshape(zero.shape[0], -1).t()], dim=-1).contiguous()


def _linear_gq_window_t_ref(x, packed, sz, *b, x_col, k, act_from_col):
    if x.device.type == "meta":
        return torch.empty((x.shape[0], packed.shape[0]), dtype=x.dtype, device="meta")
    scale = sz[..., 0].t().unsqueeze(-1)
    zero = sz[..., 1].t().unsqueeze(-1)
    return _linear_gq_window_ref(x, packed, scale, zero, *b, x_col=x_col, k=k, act_from_col=act_from_col)


OpDef("linear_gq_window_t", impl=_linear_gq_window_t_ref,
      flops=lambda op: 2 * op.attrs["k"] * op.outputs[0].nelms)


def linear_gq_window_t(x: xl.Tensor, packed: xl.Tensor, scale_zero: xl.Tensor, bias: Optional[xl.Tensor] = None,
                       x_col: int = 0, k: Optional[int] = None, act_from_col: Optional[int] = None) -> xl.Tensor:
    """`linear_gq_window` with the scales and zero points given as `interleave_scale_zero(scale, zero)`."""
    from ..xl.opdef import emit1

    k = int(k) if k is not None else x.shape[1] - x_col
    ins = [x, packed, scale_zero] + ([bias] if bias is not None else [])
    return emit1("linear_gq_window_t", ins, dict(x_col=int(x_col), k=k,
                                                 act_from_col=None if act_from_col is None else int(act_from_col)))


def linear_gq_window(x: xl.Tensor, packed: xl.Tensor, scale: xl.Tensor, zero: xl.Tensor, bias: Optional[xl.Tensor] = None,
                     x_col: int = 0, k: Optional[int] = None, act_from_col: Optional[int] = None) -> xl.Tensor:
    """`act(x[:, x_col : x_col + k] @ dequant(packed)^T + bias)` for weights quantised along the input dimension
    (`packed (out, k/gs, gs/4)`); GELU on the output columns `>= act_from_col`. Reading a column window lets one buffer
    hold the inputs of several fused layers side by side."""
    from ..xl.opdef import emit1

    k = int(k) if k is not None else x.shape[1] - x_col
    ins = [x, packed, scale, zero] + ([bias] if bias is not None else [])
    return emit1("linear_gq_window", ins, dict(x_col=int(x_col), k=k,
                                               act_from_col=None if act_from_col is None else int(act_from_col)))


class LinearGQ(Module):
    def __init__(self, out_features: int, bias: bool = True, replica_grouping: Optional[xl.ReplicaGrouping] = None,
                 group_size: int = 64, dim: int = -1):
        super().__init__()
        if group_size % 4:
            raise ValueError("group_size must be a multiple of 4")
        self.out_features = out_features
        self.bias = bias
        self.replica_grouping = replica_grouping
        self.group_size = group_size
        self.dim = dim

    def build(self, x: xl.Tensor) -> xl.Tensor:
        in_features = x.shape[-1]
        if self.dim in (-1, 1):
            u, c = in_features, self.out_features
        else:
            u, c = self.out_features, in_features
        if c % self.group_size:
            raise ValueError(f"The grouped axis ({c}) must be divisible by group_size ({self.group_size})")
        n_groups, words = c // self.group_size, self.group_size // 4
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        rg = self.replica_grouping
        packed = self.add_variable_input("weight_compressed", partial(np.zeros, (u, n_groups, words), np.uint16),
                                         xl.uint16, replica_grouping=rg)
        scale = self.add_variable_input("weight_decompression_scale", partial(np.ones, (u, n_groups, 1), np_dt),
                                        x.dtype, replica_grouping=rg)
        zero = self.add_variable_input("weight_decompression_bias", partial(np.zeros, (u, n_groups, 1), np_dt),
                                       x.dtype, replica_grouping=rg)
        ins = [x, packed, scale, zero]
        if self.bias:
            ins.append(self.add_variable_input("bias", partial(np.zeros, (self.out_features,), np_dt), x.dtype,
                                               replica_grouping=rg))
        return emit1("linear_gq", ins, {"dim": self.dim})

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, dtype: xl.dtype = xl.float32, group_size: int = 64,
                      dim: int = -1) -> WeightsDict:
        """Compress a `torch.nn.Linear` weight (stored `(out, in)`) into the layer's variables; scales, zero points
        and the bias are converted to `dtype`, the dtype of the layer's input."""
        w = nn_layer.weight.data.detach().cpu().float().numpy().T  # (in, out)
        packed, scale, bias = group_quantize_compress_numpy(w, group_size, dim)
        out = {variables.weight_compressed: packed, variables.weight_decompression_scale: to_numpy(scale, dtype),
               variables.weight_decompression_bias: to_numpy(bias, dtype)}
        if nn_layer.bias is not None and "bias" in variables:
            out[variables.bias] = to_numpy(nn_layer.bias.data, dtype)
        return WeightsDict(out)
