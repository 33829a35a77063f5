"""AdamW step for replicated tensor sharding with the three collectives folded into the update.

Given the full 16-bit weight and the full fp32 gradient accumulator of every replica in `group`, and this replica's
flat shard of the fp32 master weights, one op performs: gradient reduce-scatter (mean over the group) -> AdamW on the
shard (moments are sharded like the master weights) -> all-gather of the updated 16-bit weights into every replica's
weight. On one process per GPU with weight and accumulator placed in symmetric memory this is a single kernel that
reads its shard of each peer's accumulator and writes its shard of each peer's weight over NVLink; elsewhere it runs as
the equivalent sequence reduce-scatter, `adam_fused_`, all-gather.

The reference expresses the same step as separate graphs (rts.py:132-147 reduce, optimizers/adam.py:37-111 update,
rts.py:39-62 gather).
"""
from functools import partial
from typing import Optional

import numpy as np
import torch

from .. import xl
from ..module import Module
from ..xl.opdef import OPS, OpDef, emit1
from ..xl.ops.var_updates import _adam_fused_ref

__all__ = ["RTSAdamStep", "rts_adam_"]


def _special_rts_adam(ex, op, env):
    a = op.attrs
    w, acc, master, m, v, step = (env[t] for t in op.inputs)
    native = ex.native_collective("rts_adam")
    if native is not None:
        res = native(ex, op, w, acc, master, m, v, step)
        if res is not NotImplemented:
            env[op.outputs[0]] = w
            return
    group = a["group"]
    g_shards = ex.comm.reduce_scatter(acc, group, "mean")
    adam = OPS["adam_fused_"]
    fn = adam.native.get(ex.device.type) if ex.use_native else None
    kw = dict(has_step=True, has_master=False, bias_correction=a["bias_correction"], lr=a["lr"], beta1=a["beta1"],
              beta2=a["beta2"], epsilon=a["eps"], weight_decay=a["weight_decay"], grad_scale=a["grad_scale"],
              _tensor_scalars=())
    new = []
    for r in range(ex.num_local):
        args = (master[r], g_shards[r].reshape(master[r].shape), m[r], v[r], step[r])
        res = fn(*args, **kw) if fn is not None else NotImplemented
        if res is NotImplemented:
            adam.impl(*args, **kw)
        new.append(master[r].to(w[r].dtype))
    full = ex.comm.all_gather(new, group)
    for r in range(ex.num_local):
        w[r].copy_(full[r][: w[r].numel()].reshape(w[r].shape))
    env[op.outputs[0]] = w


OpDef("rts_adam_", special=_special_rts_adam, collective=True, inplace=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, ())])


def rts_adam_(weight: xl.Tensor, grad_accum: xl.Tensor, master_shard: xl.Tensor, first_order: xl.Tensor,
              second_order: xl.Tensor, step: xl.Tensor, group: xl.ReplicaGrouping, *, lr: float, beta1: float = 0.9,
              beta2: float = 0.999, eps: float = 1e-5, weight_decay: float = 0.0, grad_scale: float = 1.0,
              bias_correction: bool = True, sync_before: bool = True, sync_after: bool = True) -> xl.Tensor:
    """See the module docstring. `sync_before` / `sync_after`: whether this call must itself wait for all replicas'
    accumulators to be final / for all replicas' weight shards to have arrived; in a sequence of calls only the first
    needs the former and only the last the latter."""
    n = weight.nelms
    if n % group.group_size or master_shard.nelms != n // group.group_size:
        raise ValueError(f"master shard of {master_shard.nelms} elements does not match {n} / {group.group_size}")
    return emit1("rts_adam_", [weight, grad_accum, master_shard, first_order, second_order, step],
                 dict(group=group, lr=float(lr), beta1=float(beta1), beta2=float(beta2), eps=float(eps),
                      weight_decay=float(weight_decay), grad_scale=float(grad_scale),
                      bias_correction=bool(bias_correction), sync_before=bool(sync_before),
                      sync_after=bool(sync_after)))


class RTSAdamStep(Module):
    """Module form: its variables are the sharded moments and the step counter."""

    def build(self, weight: xl.TensorByRef, grad_accum: xl.Tensor, master_shard: xl.TensorByRef,
              group: xl.ReplicaGrouping, replica_grouping: Optional[xl.ReplicaGrouping] = None, *, lr: float,
              beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-5, weight_decay: float = 0.0,
              first_order_dtype: xl.dtype = xl.float32, loss_scaling: float = 1.0, bias_correction: bool = True,
              sync_before: bool = True, sync_after: bool = True):
        shape = tuple(weight.shape)
        np_m = first_order_dtype.as_numpy() if first_order_dtype._numpy is not None else np.float32
        m = self.add_replica_sharded_variable_input("first_order", partial(np.zeros, shape, np_m), first_order_dtype,
                                                    by_ref=True, replica_grouping=replica_grouping,
                                                    shard_over=group.group_size)
        v = self.add_replica_sharded_variable_input("second_order", partial(np.zeros, shape, np.float32), xl.float32,
                                                    by_ref=True, replica_grouping=replica_grouping,
                                                    shard_over=group.group_size)
        step = self.add_variable_input("step", partial(np.zeros, (), np.float32), xl.float32, by_ref=True)
        rts_adam_(weight, grad_accum, master_shard, m, v, step, group, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                  weight_decay=weight_decay, grad_scale=1.0 / float(loss_scaling), bias_correction=bias_correction,
                  sync_before=sync_before, sync_after=sync_after)
