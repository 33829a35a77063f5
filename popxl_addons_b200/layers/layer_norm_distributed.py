"""LayerNorm whose hidden axis is sharded across `replica_grouping`; each replica holds its slice of gamma/beta.
Parity: popxl_addons/layers/layer_norm_distributed.py:13-35."""
from functools import partial

from typing import Optional

import numpy as np

from .. import xl
from ..module import Module
from ..ops.layer_norm_distributed import layer_norm_distributed

__all__ = ["LayerNormDistributed"]


class LayerNormDistributed(Module):
    def __init__(self, replica_grouping: Optional[xl.ReplicaGrouping] = None, eps: float = 1e-5):
        """`replica_grouping`: the replicas the hidden axis is sharded over (default: all replicas)."""
        super().__init__()
        self._replica_grouping = replica_grouping
        self.eps = eps

    @property
    def replica_grouping(self) -> xl.ReplicaGrouping:
        return self._replica_grouping if self._replica_grouping is not None else xl.gcg().ir.replica_grouping()

    def build(self, x: xl.Tensor, eps: Optional[float] = None) -> xl.Tensor:
        """`eps` overrides the layer's own value for this graph (the reference passes it here, default 1e-5)."""
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        # parameters differ between the replicas of the group, i.e. they are identical across its transpose
        param_rg = self.replica_grouping.transpose()
        w = self.add_variable_input("weight", partial(np.ones, x.shape[-1], np_dt), x.dtype,
                                    replica_grouping=param_rg)
        b = self.add_variable_input("bias", partial(np.zeros, x.shape[-1], np_dt), x.dtype,
                                    replica_grouping=param_rg)
        return layer_norm_distributed(x, w, b, self.eps if eps is None else eps, self.replica_grouping)
