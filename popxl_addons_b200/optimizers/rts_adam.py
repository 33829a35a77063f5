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

__all__ = ["RTSAdamStep", "RTSAdamBucketStep", "rts_adam_", "rts_adam_bucket_", "rts_reduce_bucket_"]


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


# ---- buckets: many parameters per launch, optional global-norm clipping -------------------------------------------------
#
# `rts_adam_bucket_` is `rts_adam_` over a list of parameters (one kernel launch per bucket, e.g. per layer, on one
# process per GPU). For norm clipping the step is split: `rts_reduce_bucket_` leaves the group mean of the gradient in the
# owned range of each accumulator and returns the sum of squares of those ranges (what
# popxl_addons/ops/grad_reduce_square_add/grad_reduce_square_add.py:19-57 computes per tensor), the caller combines the
# sums into the global norm and a clip factor (`max_norm / max(norm, max_norm)`, popxl_addons/optimizers/adam.py:37-48),
# and `rts_adam_bucket_(..., reduced=True, scale=factor)` applies the update from the reduced gradients.


def _shard_range(ex, group, r, n_full):
    members = group.group_of(ex.global_replica(r))
    i = members.index(ex.global_replica(r))
    per = n_full // len(members)
    return i * per, per


def _special_rts_reduce_bucket(ex, op, env):
    a = op.attrs
    n = a["n"]
    accs = [env[t] for t in op.inputs[:n]]
    native = ex.native_collective("rts_reduce_bucket")
    if native is not None:
        res = native(ex, op, accs)
        if res is not NotImplemented:
            env[op.outputs[0]] = res
            return
    group = a["group"]
    sums = [torch.zeros((), dtype=torch.float32, device=accs[0][0].device) for _ in range(ex.num_local)]
    for acc in accs:
        shards = ex.comm.reduce_scatter(acc, group, "mean")
        for r in range(ex.num_local):
            off, per = _shard_range(ex, group, r, acc[r].numel())
            acc[r].reshape(-1)[off:off + per].copy_(shards[r][:per])
            sums[r] = sums[r] + (shards[r][:per].float() * a["grad_scale"]).pow(2).sum()
    env[op.outputs[0]] = sums


OpDef("rts_reduce_bucket_", special=_special_rts_reduce_bucket, collective=True, inplace=True,
      infer=lambda op: [((), xl.float32, ())])


def rts_reduce_bucket_(grad_accums, group: xl.ReplicaGrouping, grad_scale: float = 1.0, sync_before: bool = True):
    """Reduce-scatter (mean over `group`) of every accumulator of the list into its own owned range, in place; returns
    the fp32 sum of squares of `(mean * grad_scale)` over the ranges this replica owns."""
    return emit1("rts_reduce_bucket_", list(grad_accums),
                 dict(n=len(grad_accums), group=group, grad_scale=float(grad_scale), sync_before=bool(sync_before)))


def _special_rts_adam_bucket(ex, op, env):
    a = op.attrs
    n = a["n"]
    vals = [env[t] for t in op.inputs]
    ws, accs, masters, ms, vs = (vals[i * n:(i + 1) * n] for i in range(5))
    step = vals[5 * n]
    scale = vals[5 * n + 1] if a["has_scale"] else None
    native = ex.native_collective("rts_adam_bucket")
    if native is not None:
        res = native(ex, op, ws, accs, masters, ms, vs, step, scale)
        if res is not NotImplemented:
            for t, w in zip(op.outputs, ws):
                env[t] = w
            return
    group = a["group"]
    adam = OPS["adam_fused_"]
    # one step counter for the whole bucket: every parameter's update sees the advanced value, the counter advances once
    for k in range(n):
        w, acc, master, m, v = ws[k], accs[k], masters[k], ms[k], vs[k]
        if a["reduced"]:
            g_shards = []
            for r in range(ex.num_local):
                off, per = _shard_range(ex, group, r, acc[r].numel())
                g_shards.append(acc[r].reshape(-1)[off:off + per])
        else:
            g_shards = ex.comm.reduce_scatter(acc, group, "mean")
        new = []
        for r in range(ex.num_local):
            g = g_shards[r][:master[r].numel()].reshape(master[r].shape)
            if scale is not None:
                g = g * scale[r].float()
            kw = dict(has_step=True, has_master=False, bias_correction=a["bias_correction"], lr=a["lr"], beta1=a["beta1"],
                      beta2=a["beta2"], epsilon=a["eps"], weight_decay=a["weight_decays"][k], grad_scale=a["grad_scale"],
                      _tensor_scalars=())
            args = (master[r], g, m[r], v[r], step[r].clone())
            adam.impl(*args, **kw)
            new.append(master[r].to(w[r].dtype))
        full = ex.comm.all_gather(new, group)
        for r in range(ex.num_local):
            w[r].copy_(full[r][: w[r].numel()].reshape(w[r].shape))
    for r in range(ex.num_local):
        step[r].add_(1.0)
    for t, w in zip(op.outputs, ws):
        env[t] = w


OpDef("rts_adam_bucket_", special=_special_rts_adam_bucket, collective=True, inplace=True,
      infer=lambda op: [(t.shape, t.dtype, ()) for t in op.inputs[:op.attrs["n"]]])


def rts_adam_bucket_(weights, grad_accums, master_shards, first_orders, second_orders, step: xl.Tensor,
                     group: xl.ReplicaGrouping, *, lr: float, weight_decays, beta1: float = 0.9, beta2: float = 0.999,
                     eps: float = 1e-5, grad_scale: float = 1.0, bias_correction: bool = True,
                     scale: Optional[xl.Tensor] = None, reduced: bool = False, sync_before: bool = True,
                     sync_after: bool = True):
    """`rts_adam_` over lists of parameters with one shared step counter. `scale`: optional fp32 scalar tensor that
    multiplies every gradient (the clip factor); `reduced=True`: the accumulators already hold the group mean in the
    owned ranges (after `rts_reduce_bucket_`)."""
    n = len(weights)
    if not (len(grad_accums) == len(master_shards) == len(first_orders) == len(second_orders) == len(weight_decays) == n):
        raise ValueError("rts_adam_bucket_: all lists must have one entry per parameter")
    for w, mshard in zip(weights, master_shards):
        if w.nelms % group.group_size or mshard.nelms != w.nelms // group.group_size:
            raise ValueError(f"master shard of {mshard.nelms} elements does not match {w.nelms} / {group.group_size}")
    ins = [*weights, *grad_accums, *master_shards, *first_orders, *second_orders, step] + ([scale] if scale is not None else [])
    from ..xl.opdef import emit

    return emit("rts_adam_bucket_", ins,
                dict(n=n, group=group, lr=float(lr), beta1=float(beta1), beta2=float(beta2), eps=float(eps),
                     weight_decays=tuple(float(d) for d in weight_decays), grad_scale=float(grad_scale),
                     bias_correction=bool(bias_correction), has_scale=scale is not None, reduced=bool(reduced),
                     sync_before=bool(sync_before), sync_after=bool(sync_after)))


class RTSAdamBucketStep(Module):
    """Module form of `rts_adam_bucket_` for a named list of parameters: its variables are the sharded moments of every
    parameter (`<name>.first_order`, `<name>.second_order`) and one step counter."""

    def build(self, weights, grad_accums, master_shards, names, group: xl.ReplicaGrouping, replica_groupings=None, *,
              lr: float, weight_decays, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-5,
              first_order_dtype: xl.dtype = xl.float32, loss_scaling: float = 1.0, bias_correction: bool = True,
              scale: Optional[xl.Tensor] = None, reduced: bool = False, sync_before: bool = True,
              sync_after: bool = True):
        np_m = first_order_dtype.as_numpy() if first_order_dtype._numpy is not None else np.float32
        ms, vs = [], []
        rgs = replica_groupings or [None] * len(weights)
        for w, name, rg in zip(weights, names, rgs):
            shape = tuple(w.shape)
            key = name.replace(".", "_")
            ms.append(self.add_replica_sharded_variable_input(f"{key}.first_order", partial(np.zeros, shape, np_m),
                                                              first_order_dtype, by_ref=True, replica_grouping=rg,
                                                              shard_over=group.group_size, overwrite=True))
            vs.append(self.add_replica_sharded_variable_input(f"{key}.second_order", partial(np.zeros, shape, np.float32),
                                                              xl.float32, by_ref=True, replica_grouping=rg,
                                                              shard_over=group.group_size, overwrite=True))
        step = self.add_variable_input("step", partial(np.zeros, (), np.float32), xl.float32, by_ref=True)
        rts_adam_bucket_(weights, grad_accums, master_shards, ms, vs, step, group, lr=lr, weight_decays=weight_decays,
                         beta1=beta1, beta2=beta2, eps=eps, grad_scale=1.0 / float(loss_scaling),
                         bias_correction=bias_correction, scale=scale, reduced=reduced, sync_before=sync_before,
                         sync_after=sync_after)
