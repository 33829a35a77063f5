"""2-D convolution layer (NCHW).
Parity: popxl_addons/layers/conv.py:17-141. The IPU planner knobs of the reference constructor
(`available_memory_proportions`, `partials_type`, `enable_conv_dithering`) are accepted and ignored."""
from typing import Optional, Tuple, Union

from functools import partial

import numpy as np

from .. import xl
from ..utils import WeightsDict
from ..xl.utils import to_numpy
from ..module import Module
from ..named_tensors import NamedTensors
from ..xl import ops
from .linear import truncnorm_init

__all__ = ["Conv2D"]


def _pair(v) -> Tuple[int, int]:
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2D(Module):
    def __init__(self, out_channels: int, kernel_size: Union[int, Tuple[int, int]],
                 strides: Union[int, Tuple[int, int]] = (1, 1),
                 paddings: Union[str, int, Tuple[int, int], Tuple[int, int, int, int]] = (0, 0, 0, 0),
                 dilations: Union[int, Tuple[int, int]] = (1, 1), groups: int = 1, bias: bool = True,
                 available_memory_proportions=None, partials_types=None, enable_conv_dithering=None,
                 replica_grouping: Optional[xl.ReplicaGrouping] = None, cache: bool = False):
        """`paddings` is explicit `(top, left, bottom, right)` (an int or a `(vertical, horizontal)` pair are
        expanded) or one of `"same_upper"`, `"same_lower"`, `"valid"`. The three planner arguments are IPU tuning
        knobs: recorded, without effect on the values."""
        super().__init__(cache=cache)
        self.out_channels = out_channels
        self.kernel_size = _pair(kernel_size)
        self.strides = _pair(strides)
        if isinstance(paddings, str):
            if paddings not in ("not_set", "same_upper", "same_lower", "valid"):
                raise ValueError(f"Unknown padding type: {paddings}")
            self.pad_type, paddings = paddings, (0, 0, 0, 0)
        else:
            self.pad_type = "not_set"
        if isinstance(paddings, int):
            paddings = (paddings,) * 4
        elif len(paddings) == 2:
            paddings = (paddings[0], paddings[1], paddings[0], paddings[1])
        self.paddings = tuple(paddings)  # top, left, bottom, right
        self.dilations = _pair(dilations)
        self.groups = groups
        self.bias = bias
        self.replica_grouping = replica_grouping
        self.planner_hints = dict(available_memory_proportions=available_memory_proportions,
                                  partials_types=partials_types, enable_conv_dithering=enable_conv_dithering)

    def build(self, x: xl.Tensor) -> xl.Tensor:
        if x.rank != 4:
            raise ValueError(f"Conv2D expects NCHW input, got shape {x.shape}")
        in_channels = x.shape[1]
        if in_channels % self.groups or self.out_channels % self.groups:
            raise ValueError("in_channels and out_channels must be divisible by groups")
        w_shape = (self.out_channels, in_channels // self.groups, *self.kernel_size)
        w = self.add_variable_input("weight", partial(truncnorm_init, w_shape), x.dtype,
                                    replica_grouping=self.replica_grouping)
        y = ops.conv(x, w, stride=self.strides, padding=self.paddings, dilation=self.dilations, groups=self.groups,
                     pad_type=self.pad_type, **self.planner_hints)
        if self.bias:
            b = self.add_variable_input("bias", partial(np.zeros, (1, self.out_channels, 1, 1)), x.dtype,
                                        replica_grouping=self.replica_grouping)
            y = y + b
        return y

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, dtype: xl.dtype = xl.float32) -> WeightsDict:
        out = {variables.weight: to_numpy(nn_layer.weight.data, dtype)}
        if nn_layer.bias is not None and "bias" in variables:
            out[variables.bias] = to_numpy(nn_layer.bias.data, dtype).reshape(variables.bias.shape)
        return WeightsDict(out)
