"""2-D convolution layer (NCHW).
Parity: popxl_addons/layers/conv.py:17-141. The IPU planner knobs of the reference constructor
(`available_memory_proportions`, `partials_type`, `enable_conv_dithering`) are accepted and ignored."""
from typing import Dict, Iterable, Optional, Tuple, Union

import numpy as np

from .. import xl
from ..module import Module
from ..named_tensors import NamedTensors
from ..xl import ops

__all__ = ["Conv2D"]


def _pair(v) -> Tuple[int, int]:
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2D(Module):
    def __init__(self, out_channels: int, kernel_size: Union[int, Tuple[int, int]],
                 strides: Union[int, Tuple[int, int]] = 1,
                 paddings: Union[int, Tuple[int, int], Tuple[int, int, int, int]] = 0,
                 dilations: Union[int, Tuple[int, int]] = 1, groups: int = 1, bias: bool = True,
                 pad_type: str = "not_set", available_memory_proportions=None, partials_type=None,
                 enable_conv_dithering=None, replica_grouping: Optional[xl.ReplicaGrouping] = None,
                 cache: bool = False):
        super().__init__(cache=cache)
        self.out_channels = out_channels
        self.kernel_size = _pair(kernel_size)
        self.strides = _pair(strides)
        if isinstance(paddings, int):
            paddings = (paddings,) * 4
        elif len(paddings) == 2:
            paddings = (paddings[0], paddings[1], paddings[0], paddings[1])
        self.paddings = tuple(paddings)  # top, left, bottom, right
        self.dilations = _pair(dilations)
        self.groups = groups
        self.bias = bias
        if pad_type not in ("not_set", "same_upper", "same_lower", "valid"):
            raise ValueError(f"Unknown pad_type: {pad_type}")
        self.pad_type = pad_type
        self.replica_grouping = replica_grouping

    def build(self, x: xl.Tensor) -> xl.Tensor:
        if x.rank != 4:
            raise ValueError(f"Conv2D expects NCHW input, got shape {x.shape}")
        in_channels = x.shape[1]
        if in_channels % self.groups or self.out_channels % self.groups:
            raise ValueError("in_channels and out_channels must be divisible by groups")
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w_shape = (self.out_channels, in_channels // self.groups, *self.kernel_size)
        fan_in = int(np.prod(w_shape[1:]))
        bound = 1.0 / np.sqrt(fan_in)
        w = self.add_variable_input("weight", lambda: np.random.uniform(-bound, bound, w_shape).astype(np_dt),
                                    x.dtype, replica_grouping=self.replica_grouping)
        y = ops.conv(x, w, stride=self.strides, padding=self.paddings, dilation=self.dilations, groups=self.groups,
                     pad_type=self.pad_type)
        if self.bias:
            b = self.add_variable_input("bias", lambda: np.random.uniform(-bound, bound, self.out_channels)
                                        .astype(np_dt), x.dtype, replica_grouping=self.replica_grouping)
            y = y + b.reshape((1, self.out_channels, 1, 1))
        return y

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer) -> Dict[xl.Tensor, np.ndarray]:
        out = {variables.weight: nn_layer.weight.data.detach().cpu().numpy().copy()}
        if nn_layer.bias is not None and "bias" in variables:
            out[variables.bias] = nn_layer.bias.data.detach().cpu().numpy().copy()
        return out
