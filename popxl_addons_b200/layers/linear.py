"""Dense layer `y = x @ w + b` with weight shape `(in, out)`.

With a `replica_grouping` whose groups are smaller than the replica set the weights differ between groups, which is
how column/row tensor-parallel shards are declared (identical across the data-parallel group, different across the
tensor-parallel one).
Parity: popxl_addons/layers/linear.py:17-65.
"""
from functools import partial
from typing import Optional

import numpy as np

from .. import xl
from ..utils import WeightsDict
from ..xl.utils import to_numpy
from ..module import Module
from ..named_tensors import NamedTensors

__all__ = ["Linear", "truncnorm_init"]


def truncnorm_init(shape, std: float = 0.02, dtype=np.float32) -> np.ndarray:
    """Normal(0, std) truncated at two standard deviations."""
    from scipy.stats import truncnorm

    return truncnorm.rvs(-2, 2, loc=0, scale=std, size=tuple(shape)).astype(dtype)


class Linear(Module):
    def __init__(self, out_features: int, bias: bool = True,
                 replica_grouping: Optional[xl.ReplicaGrouping] = None, cache: bool = False):
        super().__init__(cache=cache)
        self.out_features = out_features
        self.bias = bias
        self.replica_grouping = replica_grouping

    def build(self, x: xl.Tensor) -> xl.Tensor:
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w = self.add_variable_input("weight", partial(truncnorm_init, (x.shape[-1], self.out_features), 0.02, np_dt),
                                    x.dtype, replica_grouping=self.replica_grouping)
        y = x @ w
        if self.bias:
            b = self.add_variable_input("bias", partial(np.zeros, (self.out_features,), np_dt), x.dtype,
                                        replica_grouping=self.replica_grouping)
            y = y + b
        return y

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, dtype: xl.dtype = xl.float32) -> WeightsDict:
        """Host data for `variables` from a `torch.nn.Linear` (whose weight is `(out, in)`), converted to `dtype`."""
        out = {variables.weight: np.ascontiguousarray(to_numpy(nn_layer.weight.data, dtype).T)}
        if nn_layer.bias is not None and "bias" in variables:
            out[variables.bias] = to_numpy(nn_layer.bias.data, dtype)
        return WeightsDict(out)
