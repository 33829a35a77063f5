"""LayerNorm over the last axis of a 2-D `(N, C)` tensor.
Parity: popxl_addons/layers/layer_norm.py:14-54."""
from functools import partial
from typing import Optional

import numpy as np

from .. import xl
from ..utils import WeightsDict
from ..xl.utils import to_numpy
from ..module import Module
from ..named_tensors import NamedTensors
from ..xl import ops

__all__ = ["LayerNorm"]


class LayerNorm(Module):
    def __init__(self, eps: float = 1e-5, cache: bool = False):
        super().__init__(cache=cache)
        self.eps = eps

    def build(self, x: xl.Tensor, eps: Optional[float] = None) -> xl.Tensor:
        """`eps` overrides the layer's own value for this graph (the reference passes it here, default 1e-5)."""
        if x.rank != 2:
            raise ValueError(f"LayerNorm expects a 2-D (N, C) input; got shape {x.shape}. Flatten leading axes first.")
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w = self.add_variable_input("weight", partial(np.ones, x.shape[-1], np_dt), x.dtype)
        b = self.add_variable_input("bias", partial(np.zeros, x.shape[-1], np_dt), x.dtype)
        return ops.layer_norm(x, w, b, eps=self.eps if eps is None else eps)

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, dtype: xl.dtype = xl.float32) -> WeightsDict:
        """A torch LayerNorm over several trailing axes maps onto this layer's flattened last axis."""
        return WeightsDict({variables.weight: to_numpy(nn_layer.weight.data, dtype).reshape(variables.weight.shape),
                            variables.bias: to_numpy(nn_layer.bias.data, dtype).reshape(variables.bias.shape)})
