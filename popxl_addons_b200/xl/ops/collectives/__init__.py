"""Replica collectives (`xl.ops.collectives.*`): all-reduce, reduce-scatter, all-gather and the local shard slice.

A collective runs over the groups of a `ReplicaGrouping`; at run time the session's communicator carries it out: an
in-process exchange when all replicas are simulated in one process, NCCL or the package's own NVLink kernels when
there is one process per GPU.
Parity: popxl `ops.collectives.{replicated_all_reduce, replicated_reduce_scatter, replicated_all_gather,
replica_sharded_slice}` (rts.py:58,136-145) and the autograd pairings of
ops/replicated_all_reduce_TP/replicated_all_reduce_TP_binding.cpp:82-100.
"""
from typing import Optional

import numpy as np

from ...core import ReplicaGrouping, Tensor, gcg
from ...opdef import OpDef, emit, emit1

_REDUCE_OPS = ("add", "mean", "max", "min", "mul")


def _group(group: Optional[ReplicaGrouping]) -> ReplicaGrouping:
    return group if group is not None else gcg().ir.replica_grouping()


def _norm_op(op) -> str:
    name = getattr(op, "name", op)
    name = str(name).lower()
    if name not in _REDUCE_OPS:
        raise ValueError(f"Unsupported collective operator: {op}. Supported: {_REDUCE_OPS}")
    return name


# ---- all-reduce ----------------------------------------------------------------------------------------------


def _special_all_reduce(ex, op, env):
    if op.attrs.get("identical_inputs"):
        raise RuntimeError(
            "An all-reduce with identical inputs is an identity in the forward pass: run "
            "`apply_pre_alias_patterns(ir)` (OpToIdentityPattern) before creating the session.")
    vals = env[op.inputs[0]]
    env[op.outputs[0]] = ex.comm.all_reduce(vals, op.attrs["group"], op.attrs["op"], inplace=op.attrs["inplace"],
                                            async_ok=True)


def _vjp_all_reduce(ctx, op, gs):
    a = op.attrs
    if a["op"] not in ("add", "mean"):
        raise NotImplementedError("Only add/mean all-reduce is differentiable")
    if a.get("identical_grad_inputs"):
        # forward all-reduce / backward identity (Megatron g)
        return [gs[0]]
    if a.get("identical_inputs"):
        # forward identity / backward all-reduce (Megatron f)
        return [emit1("all_reduce", [gs[0]], dict(group=a["group"], op=a["op"], inplace=False,
                                                  identical_inputs=False, identical_grad_inputs=True))]
    return [emit1("all_reduce", [gs[0]], dict(group=a["group"], op=a["op"], inplace=False,
                                              identical_inputs=False, identical_grad_inputs=False))]


OpDef("all_reduce", special=_special_all_reduce, vjp=_vjp_all_reduce, collective=True, keeps_meta=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, op.inputs[0].meta_shape)])


def replicated_all_reduce(t: Tensor, op="add", group: Optional[ReplicaGrouping] = None,
                          identical_inputs: bool = False, identical_grad_inputs: bool = False,
                          inplace: bool = False) -> Tensor:
    if identical_inputs and identical_grad_inputs:
        raise ValueError("`identical_inputs` and `identical_grad_inputs` cannot both be set")
    return emit1("all_reduce", [t], dict(group=_group(group), op=_norm_op(op), inplace=inplace,
                                         identical_inputs=identical_inputs,
                                         identical_grad_inputs=identical_grad_inputs))


def replicated_all_reduce_(t: Tensor, op="add", group: Optional[ReplicaGrouping] = None) -> Tensor:
    return replicated_all_reduce(t, op, group, inplace=True)


# ---- reduce-scatter ------------------------------------------------------------------------------------------


def _shard_len(nelms: int, size: int) -> int:
    return -(-nelms // size)


def _special_reduce_scatter(ex, op, env):
    env[op.outputs[0]] = ex.comm.reduce_scatter(env[op.inputs[0]], op.attrs["group"], op.attrs["op"])


def _infer_reduce_scatter(op):
    t = op.inputs[0]
    n = _shard_len(t.nelms, op.attrs["group"].group_size)
    meta = tuple(t.shape) if op.attrs["rts"] else ()
    return [((n,), t.dtype, meta)]


def _vjp_reduce_scatter(ctx, op, gs):
    t = op.inputs[0]
    full = emit1("all_gather", [gs[0]], dict(group=op.attrs["group"]))
    if full.nelms != t.nelms:
        from .. import slice as _slice

        full = _slice(full, [0], [t.nelms], [1], [0])
    from .. import reshape

    return [reshape(full, t.shape)]


OpDef("reduce_scatter", special=_special_reduce_scatter, infer=_infer_reduce_scatter, vjp=_vjp_reduce_scatter,
      collective=True)


def replicated_reduce_scatter(t: Tensor, op="add", group: Optional[ReplicaGrouping] = None,
                              configure_output_for_replicated_tensor_sharding: bool = False) -> Tensor:
    """Reduce over the group and keep this replica's `ceil(nelms/size)` slice of the flattened result (zero padded).
    With `configure_output_for_replicated_tensor_sharding` the output remembers the input shape as `meta_shape`."""
    return emit1("reduce_scatter", [t], dict(group=_group(group), op=_norm_op(op),
                                             rts=bool(configure_output_for_replicated_tensor_sharding)))


# ---- all-gather ----------------------------------------------------------------------------------------------


def _special_all_gather(ex, op, env):
    env[op.outputs[0]] = ex.comm.all_gather(env[op.inputs[0]], op.attrs["group"])


def _infer_all_gather(op):
    t = op.inputs[0]
    return [((t.nelms * op.attrs["group"].group_size,), t.dtype, ())]


def _vjp_all_gather(ctx, op, gs):
    g = emit1("reduce_scatter", [gs[0]], dict(group=op.attrs["group"], op="add", rts=False))
    from .. import reshape

    return [reshape(g, op.inputs[0].shape)]


OpDef("all_gather", special=_special_all_gather, infer=_infer_all_gather, vjp=_vjp_all_gather, collective=True)


def replicated_all_gather(t: Tensor, group: Optional[ReplicaGrouping] = None, output_shape=None) -> Tensor:
    """Concatenate the flattened shards of the group in group order. The result is reshaped to the shard's
    `meta_shape` when it has one (or to `output_shape`)."""
    out = emit1("all_gather", [t], dict(group=_group(group)))
    target = tuple(output_shape) if output_shape is not None else (t.meta_shape or None)
    if target:
        from .. import reshape

        out = reshape(out, target)
    return out


# ---- local slice ---------------------------------------------------------------------------------------------


def _special_sharded_slice(ex, op, env):
    group: ReplicaGrouping = op.attrs["group"]
    n = op.outputs[0].nelms
    outs = []
    for r, v in enumerate(env[op.inputs[0]]):
        i = group.index_in_group(ex.global_replica(r))
        outs.append(v.reshape(-1)[i * n:(i + 1) * n].clone())
    env[op.outputs[0]] = outs


def _infer_sharded_slice(op):
    t = op.inputs[0]
    size = op.attrs["group"].group_size
    if t.nelms % size != 0:
        raise ValueError(f"Cannot slice {t.nelms} elements into {size} equal shards")
    return [((t.nelms // size,), t.dtype, tuple(t.shape))]


OpDef("replica_sharded_slice", special=_special_sharded_slice, infer=_infer_sharded_slice, collective=True)


def replica_sharded_slice(t: Tensor, group: Optional[ReplicaGrouping] = None) -> Tensor:
    """This replica's flat shard of `t` (no communication): position in `group` selects the slice."""
    grp = _group(group)
    if grp.group_size == 1:
        return t
    return emit1("replica_sharded_slice", [t], dict(group=grp))


replicated_slice = replica_sharded_slice


# ---- forward-identity half of the tensor-parallel all-reduce (result of the OpToIdentity rewrite) -------------


def _vjp_tp_identity(ctx, op, gs):
    return [emit1("all_reduce", [gs[0]], dict(group=op.attrs["group"], op=op.attrs["op"], inplace=False,
                                              identical_inputs=False, identical_grad_inputs=True))]


OpDef("tp_identity", impl=lambda a, **kw: a, vjp=_vjp_tp_identity, keeps_meta=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, op.inputs[0].meta_shape)])


# ---- all-reduce over the device slots of one replica ---------------------------------------------------------------


def _slot_all_reduce_ref(*ts, op, identity, mode=None):
    if identity:
        return tuple(ts)
    import torch

    stacked = torch.stack([t.to(ts[0].device).float() for t in ts])
    red = {"add": stacked.sum(0), "mean": stacked.mean(0), "max": stacked.amax(0), "min": stacked.amin(0),
           "mul": stacked.prod(0)}[op]
    return tuple(red.to(device=t.device, dtype=t.dtype) for t in ts)


def _vjp_slot_all_reduce(ctx, op, gs):
    a = op.attrs
    if a["op"] not in ("add", "mean"):
        raise NotImplementedError("Only add/mean all-reduce is differentiable")
    from .. import init

    gs = [g if g is not None else init(o.shape, o.dtype, "zero_grad", "zero") for g, o in zip(gs, op.outputs)]
    mode = a["mode"]
    if mode == "identical_grad_inputs":  # forward all-reduce / backward identity
        return list(gs)
    back = "identical_grad_inputs" if mode == "identical_inputs" else "both"
    return list(emit("slot_all_reduce", gs, dict(op=a["op"], mode=back, identity=False)))


OpDef("slot_all_reduce", impl=_slot_all_reduce_ref, vjp=_vjp_slot_all_reduce,
      infer=lambda op: [(t.shape, t.dtype, t.meta_shape) for t in op.inputs])


def _slot_all_reduce(ts, operation, ipus, mode):
    ts = list(ts)
    if not ts:
        raise ValueError("all_reduce needs at least one tensor")
    if ipus is not None and len(list(ipus)) != len(ts):
        raise ValueError("Number of specified IPUs does not equal number of input tensors")
    if any(t.shape != ts[0].shape or t.dtype != ts[0].dtype for t in ts):
        raise ValueError("all_reduce takes tensors of one shape and dtype")
    if gcg().ir.devices_per_replica > 1:
        raise NotImplementedError(
            "With one process per device slot an all-reduce over the slots of a replica has no single launching "
            "process: shard over replicas instead (a tensor-parallel ReplicaGrouping and `replicated_all_reduce`).")
    return tuple(emit("slot_all_reduce", ts, dict(op=_norm_op(operation), mode=mode,
                                                  identity=(mode == "identical_inputs"))))


def all_reduce(ts, operation="add", ipus=None):
    """All-reduce the tensors `ts`, one per device slot (`ipu(i)`) of a replica; returns the reduced value once per
    input. The backward pass all-reduces the gradients."""
    return _slot_all_reduce(ts, operation, ipus, "both")


def all_reduce_identical_inputs(ts, operation="add", ipus=None):
    """Identity in the forward pass (the inputs are known to be equal), all-reduce of the gradients in the backward
    pass."""
    return _slot_all_reduce(ts, operation, ipus, "identical_inputs")


def all_reduce_identical_grad_inputs(ts, operation="add", ipus=None):
    """All-reduce in the forward pass, identity in the backward pass (the gradients are known to be equal)."""
    return _slot_all_reduce(ts, operation, ipus, "identical_grad_inputs")
