"""AdamW step as a Module: its variables are the optimizer state, so state is created, sharded, checkpointed and
offloaded exactly like model weights.

If the variable to update is a replica shard (has a `meta_shape`), the state is created with the same sharding
(flat shards over the same number of replicas). By default the whole step is emitted as one fused op (one kernel on
CUDA); `fused=False` emits the reference's op sequence (moving averages, `adam_updater`, `scaled_add_`).
Parity: popxl_addons/optimizers/adam.py:14-111.
"""
from functools import partial
from typing import Optional, Union

import numpy as np

from .. import xl
from ..module import Module
from ..xl import ops

__all__ = ["AdamOptimizerStep"]

Scalar = Union[float, xl.Tensor]


class AdamOptimizerStep(Module):
    def __init__(self, cache: bool = False, fused: bool = True):
        super().__init__(cache=cache)
        self.fused = fused

    def _state(self, name: str, var: xl.Tensor, dtype: xl.dtype, replica_grouping):
        np_dt = dtype.as_numpy() if dtype._numpy is not None else np.float32
        if var.meta_shape:
            shard_over = int(np.prod(var.meta_shape)) // int(np.prod(var.shape))
            return self.add_replica_sharded_variable_input(
                name, partial(np.zeros, var.meta_shape, np_dt), dtype, by_ref=True,
                replica_grouping=replica_grouping, shard_over=shard_over)
        return self.add_variable_input(name, partial(np.zeros, var.shape, np_dt), dtype, by_ref=True,
                                       replica_grouping=replica_grouping)

    def build(self, var: xl.TensorByRef, grad: xl.Tensor, replica_grouping: Optional[xl.ReplicaGrouping] = None, *,
              lr: Scalar, beta1: Scalar = 0.9, beta2: Scalar = 0.999, eps: Scalar = 1e-5,
              weight_decay: Scalar = 1e-2, first_order_dtype: xl.dtype = xl.float16, bias_correction: bool = True,
              loss_scaling: Scalar = 1, global_norm: Optional[xl.Tensor] = None,
              global_norm_max: Optional[Scalar] = None, master: Optional[xl.Tensor] = None):
        """Update `var` in place with gradient `grad`. `loss_scaling` divides the gradient; with `global_norm` and
        `global_norm_max` it is additionally scaled by `max_norm / max(global_norm, max_norm)` (norm clipping).
        `master` is an optional fp32 copy of `var` that receives the update at full precision."""
        if isinstance(loss_scaling, xl.Tensor):
            scale = ops.div(xl.constant(1.0, xl.float32), ops.cast(loss_scaling, xl.float32))
        else:
            scale = 1.0 / float(loss_scaling)
        if global_norm is not None and global_norm_max is not None:
            gmax = global_norm_max if isinstance(global_norm_max, xl.Tensor) else xl.constant(
                float(global_norm_max), xl.float32)
            clip = ops.div(gmax, ops.maximum(ops.cast(global_norm, xl.float32), gmax))
            scale = ops.mul(clip, scale if isinstance(scale, xl.Tensor) else xl.constant(scale, xl.float32))
        first_order = self._state("first_order", var, first_order_dtype, replica_grouping)
        second_order = self._state("second_order", var, xl.float32, replica_grouping)
        step = None
        if bias_correction:
            step = self.add_variable_input("step", partial(np.zeros, (), np.float32), xl.float32, by_ref=True)
        if self.fused:
            ops.var_updates.adam_fused_(var, grad, first_order, second_order, step, master, lr=lr, beta1=beta1,
                                        beta2=beta2, epsilon=eps, weight_decay=weight_decay, grad_scale=scale,
                                        bias_correction=bias_correction)
            return
        g = ops.cast(grad, xl.float32)
        g = ops.mul(g, scale) if isinstance(scale, xl.Tensor) else (g * scale if scale != 1.0 else g)
        ops.var_updates.accumulate_moving_average_(first_order, g, f=beta1)
        ops.var_updates.accumulate_moving_average_square_(second_order, g, f=beta2)
        target = master if master is not None else var
        updater = ops.var_updates.adam_updater(first_order, second_order, weight=target, weight_decay=weight_decay,
                                               time_step=step, beta1=beta1 if step is not None else None,
                                               beta2=beta2 if step is not None else None, epsilon=eps)
        neg_lr = ops.negate(lr) if isinstance(lr, xl.Tensor) else -float(lr)
        ops.scaled_add_(target, updater, b=neg_lr)
        if master is not None:
            ops.var_updates.copy_var_update_(var, ops.cast(master, var.dtype))
