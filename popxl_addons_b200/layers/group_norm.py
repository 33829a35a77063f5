"""GroupNorm over channel axis 1.
Parity: popxl_addons/layers/group_norm.py:16-68."""
from functools import partial
from typing import Optional

import numpy as np

from .. import xl
from ..utils import WeightsDict
from ..xl.utils import to_numpy
from ..module import Module
from ..named_tensors import NamedTensors
from ..xl import ops

__all__ = ["GroupNorm"]


class GroupNorm(Module):
    def __init__(self, num_groups: int, replica_grouping: Optional[xl.ReplicaGrouping] = None, eps: float = 1e-5,
                 cache: bool = False):
        super().__init__(cache=cache)
        self.num_groups = num_groups
        self.replica_grouping = replica_grouping
        self.eps = eps

    def build(self, x: xl.Tensor) -> xl.Tensor:
        c = x.shape[1]
        if c % self.num_groups:
            raise ValueError(f"{c} channels are not divisible into {self.num_groups} groups")
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w = self.add_variable_input("weight", partial(np.ones, c, np_dt), x.dtype,
                                    replica_grouping=self.replica_grouping)
        b = self.add_variable_input("bias", partial(np.zeros, c, np_dt), x.dtype,
                                    replica_grouping=self.replica_grouping)
        return ops.group_norm(x, w, b, num_groups=self.num_groups, eps=self.eps)

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, dtype: xl.dtype = xl.float32) -> WeightsDict:
        return WeightsDict({variables.weight: to_numpy(nn_layer.weight.data, dtype),
                            variables.bias: to_numpy(nn_layer.bias.data, dtype)})
