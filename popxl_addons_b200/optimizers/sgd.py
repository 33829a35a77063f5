"""SGD step (optional momentum and L2 weight decay) with the same Module shape as `AdamOptimizerStep`.

`g' = g / loss_scaling + wd * w ; buf = momentum * buf + g' ; w -= lr * buf`. The reference ships Adam only (its
MNIST test does the plain update by hand with `scaled_add_`, tests/integration/test_mnist_fp8.py:167-212).
"""
from functools import partial
from typing import Optional, Union

import numpy as np

from .. import xl
from ..module import Module
from ..xl import ops

__all__ = ["SGDOptimizerStep"]

Scalar = Union[float, xl.Tensor]


class SGDOptimizerStep(Module):
    def build(self, var: xl.TensorByRef, grad: xl.Tensor, replica_grouping: Optional[xl.ReplicaGrouping] = None, *,
              lr: Scalar, momentum: Scalar = 0.0, weight_decay: Scalar = 0.0, loss_scaling: Scalar = 1,
              momentum_dtype: xl.dtype = xl.float32):
        if isinstance(loss_scaling, xl.Tensor):
            scale = ops.div(xl.constant(1.0, xl.float32), ops.cast(loss_scaling, xl.float32))
        else:
            scale = 1.0 / float(loss_scaling)
        buf = None
        if isinstance(momentum, xl.Tensor) or momentum != 0.0:
            np_dt = momentum_dtype.as_numpy() if momentum_dtype._numpy is not None else np.float32
            if var.meta_shape:
                shard_over = int(np.prod(var.meta_shape)) // int(np.prod(var.shape))
                buf = self.add_replica_sharded_variable_input(
                    "momentum", partial(np.zeros, var.meta_shape, np_dt), momentum_dtype, by_ref=True,
                    replica_grouping=replica_grouping, shard_over=shard_over)
            else:
                buf = self.add_variable_input("momentum", partial(np.zeros, var.shape, np_dt), momentum_dtype,
                                              by_ref=True, replica_grouping=replica_grouping)
        ops.var_updates.sgd_fused_(var, grad, buf, lr=lr, momentum=momentum, weight_decay=weight_decay,
                                   grad_scale=scale)
