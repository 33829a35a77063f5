"""Cross-entropy with the class (vocabulary) axis sharded over a tensor-parallel replica group.

Per row: group max -> `exp(x - max)` -> group sum -> `-(x - max - log sum)` (negative log-softmax of the local slice)
-> pick the label's entry if it falls in this shard (else 0) -> group sum. Three reductions of `n_samples` values
cross the group. The gradient is `softmax * dL` with `dL` subtracted at the label position, local to each shard.
`cross_entropy_sharded_wr_loss` is the variant with uneven shards, un-offset indices and the loss delivered on the
first shard only (model parallelism inside one replica in the reference).

Parity: popxl_addons/ops/cross_entropy_sharded_loss/cross_entropy_sharded_loss.py:26-98 (+ crossentropyshardedx.cpp
:88-298) and ops/cross_entropy_sharded_wr_loss/cross_entropy_sharded_wr_loss.py:40-89.
"""
from typing import Iterable, List, Optional

import torch

from .. import xl
from ..xl import ops
from ..xl.opdef import OpDef, emit

__all__ = ["cross_entropy_sharded_loss", "cross_entropy_sharded_wr_loss", "cross_entropy_sharded_with_grad"]


def _local_stats(logits: torch.Tensor):
    return logits.float().amax(dim=-1)


def _special_ce_fwd(ex, op, env):
    group = op.attrs["group"]
    logits, idx = env[op.inputs[0]], env[op.inputs[1]]
    native = ex.native_collective("ce_sharded_fwd")
    if native is not None:
        res = native(ex, op, logits, idx)
        if res is not NotImplemented:
            env[op.outputs[0]], env[op.outputs[1]] = res
            return
    local_max = [l.float().amax(dim=-1) for l in logits]
    gmax = ex.comm.all_reduce(local_max, group, "max")
    shifted = [l.float() - m.unsqueeze(-1) for l, m in zip(logits, gmax)]
    local_sum = [torch.exp(s).sum(dim=-1) for s in shifted]
    gsum = ex.comm.all_reduce(local_sum, group, "add")
    nls = [-(s - torch.log(z).unsqueeze(-1)) for s, z in zip(shifted, gsum)]
    picked = []
    for n, i in zip(nls, idx):
        il = i.long()
        ok = (il >= 0) & (il < n.shape[-1])
        picked.append(n.gather(1, il.clamp(0, n.shape[-1] - 1).unsqueeze(1)).squeeze(1) * ok.float())
    loss = ex.comm.all_reduce(picked, group, "add")
    dt = logits[0].dtype
    env[op.outputs[0]] = [l.to(dt) for l in loss]
    env[op.outputs[1]] = [n.to(dt) for n in nls]


def _ce_bwd_ref(nls, idx, dloss):
    if nls.device.type == "meta":
        return torch.empty_like(nls)
    g = torch.exp(-nls.float()) * dloss.float().unsqueeze(-1)
    il = idx.long()
    ok = (il >= 0) & (il < nls.shape[-1])
    sub = torch.zeros_like(g)
    sub.scatter_(1, il.clamp(0, nls.shape[-1] - 1).unsqueeze(1), (dloss.float() * ok.float()).unsqueeze(1))
    return (g - sub).to(nls.dtype)


def _vjp_ce(ctx, op, gs):
    nls = ctx.fwd(op.outputs[1])
    idx = ctx.fwd(op.inputs[1])
    return [emit("ce_sharded_grad", [nls, idx, gs[0]])[0], None]


def _special_ce_with_grad(ex, op, env):
    """`(loss per row, dlogits)` from `(logits, labels, per-row loss gradient)` in one op: the softmax is never kept."""
    group = op.attrs["group"]
    logits, idx, dl = env[op.inputs[0]], env[op.inputs[1]], env[op.inputs[2]]
    native = ex.native_collective("ce_sharded_with_grad")
    if native is not None:
        res = native(ex, op, logits, idx, dl)
        if res is not NotImplemented:
            dt = logits[0].dtype
            env[op.outputs[0]] = [r.to(dt) for r in res[0]]
            env[op.outputs[1]] = res[1]
            return
    local_max = [l.float().amax(dim=-1) for l in logits]
    gmax = ex.comm.all_reduce(local_max, group, "max")
    shifted = [l.float() - m.unsqueeze(-1) for l, m in zip(logits, gmax)]
    gsum = ex.comm.all_reduce([torch.exp(s).sum(dim=-1) for s in shifted], group, "add")
    picked, hot = [], []
    for s, i in zip(shifted, idx):
        il = i.long()
        ok = (il >= 0) & (il < s.shape[-1])
        picked.append(s.gather(1, il.clamp(0, s.shape[-1] - 1).unsqueeze(1)).squeeze(1) * ok.float())
        hot.append((il.clamp(0, s.shape[-1] - 1), ok))
    gpicked = ex.comm.all_reduce(picked, group, "add")
    dt = logits[0].dtype
    env[op.outputs[0]] = [(torch.log(z) - p).to(dt) for z, p in zip(gsum, gpicked)]
    grads = []
    for s, z, d, (il, ok) in zip(shifted, gsum, dl, hot):
        g = torch.exp(s) / z.unsqueeze(-1)
        g.scatter_add_(1, il.unsqueeze(1), -ok.float().unsqueeze(1))
        grads.append((g * d.float().unsqueeze(-1)).to(dt))
    env[op.outputs[1]] = grads


OpDef("ce_sharded_with_grad", special=_special_ce_with_grad, collective=True,
      infer=lambda op: [((op.inputs[0].shape[0],), op.inputs[0].dtype, ()),
                        (op.inputs[0].shape, op.inputs[0].dtype, ())])
OpDef("ce_sharded", special=_special_ce_fwd, vjp=_vjp_ce, collective=True,
      infer=lambda op: [((op.inputs[0].shape[0],), op.inputs[0].dtype, ()),
                        (op.inputs[0].shape, op.inputs[0].dtype, ())])
OpDef("ce_sharded_grad", impl=_ce_bwd_ref)


def _reduce_loss(loss, indices, ignore_index, reduction):
    mask = None
    if ignore_index is not None:
        ii = ignore_index if isinstance(ignore_index, xl.Tensor) else xl.constant(ignore_index, indices.dtype)
        mask = ops.cast(ops.logical_not(ops.equal(indices, ii)), loss.dtype)
        loss = loss * mask
    if reduction == "mean":
        return ops.sum(loss) / ops.sum(mask) if mask is not None else ops.mean(loss)
    if reduction == "sum":
        return ops.sum(loss)
    if reduction != "none":
        raise ValueError(f"`reduction` should be one of `mean`, `sum` and `none`. Passed: {reduction}")
    return loss


def cross_entropy_sharded_loss(logits: xl.Tensor, indices: xl.Tensor, ignore_index=None,
                               replica_grouping: Optional[xl.ReplicaGrouping] = None, reduction: str = "mean",
                               available_memory_proportion: float = 0.4) -> xl.Tensor:
    """`logits (n_samples, classes/tp)` differ per replica of the group; `indices (n_samples,)` are identical on
    all replicas *before* each replica subtracts its shard offset (the caller does that), so out-of-shard labels are
    out of range locally. `ignore_index` must be offset the same way. The loss is identical on all replicas."""
    if logits.rank != 2:
        raise ValueError(f"logits must be 2-D (n_samples, sharded_n_classes), got {logits.shape}")
    if indices.rank != 1 or indices.shape[0] != logits.shape[0]:
        raise ValueError(f"indices must have shape ({logits.shape[0]},), got {indices.shape}")
    group = replica_grouping if replica_grouping is not None else xl.gcg().ir.replica_grouping()
    loss, _ = emit("ce_sharded", [logits, indices], {"group": group, "root_only": False},
                   ["cross_entropy_sharded_out", "cross_entropy_sharded_soft_max_out"])
    return _reduce_loss(loss, indices, ignore_index, reduction)


def cross_entropy_sharded_with_grad(logits: xl.Tensor, indices: xl.Tensor, loss_scaling=1.0, ignore_index=None,
                                    replica_grouping: Optional[xl.ReplicaGrouping] = None, reduction: str = "mean"):
    """Vocabulary-sharded counterpart of `cross_entropy_with_grad`: returns `(loss, d(loss*loss_scaling)/dlogits)`
    where the gradient is this replica's slice. No separate backward graph is needed for the loss."""
    group = replica_grouping if replica_grouping is not None else xl.gcg().ir.replica_grouping()
    n = logits.shape[0]
    scale = loss_scaling if isinstance(loss_scaling, xl.Tensor) else xl.constant(float(loss_scaling), xl.float32)
    if ignore_index is not None:
        ii = ignore_index if isinstance(ignore_index, xl.Tensor) else xl.constant(ignore_index, indices.dtype)
        mask = ops.cast(ops.logical_not(ops.equal(indices, ii)), xl.float32)
    else:
        mask = None
    if reduction == "mean":
        denom = ops.sum(mask) if mask is not None else xl.constant(float(n), xl.float32)
        per_row = ops.div(scale, denom)
    elif reduction in ("sum", "none"):
        per_row = scale
    else:
        raise ValueError(f"`reduction` should be one of `mean`, `sum` and `none`. Passed: {reduction}")
    dl = ops.expand(ops.reshape(per_row, (1,)), (n,)) if per_row.shape == () else per_row
    if mask is not None:
        dl = dl * mask
    dl = ops.cast(dl, xl.float32)
    rows, dlogits = emit("ce_sharded_with_grad", [logits, indices, dl], {"group": group},
                         ["cross_entropy_sharded_out", "cross_entropy_sharded_grad"])
    return _reduce_loss(rows, indices, ignore_index, reduction), dlogits


# ---- variant: all shards are tensors of one replica -----------------------------------------------------------


def _ce_wr_fwd_ref(*tensors, n):
    logits, indices = tensors[:n], tensors[n:]
    if logits[0].device.type == "meta":
        return (torch.empty((logits[0].shape[0],), dtype=logits[0].dtype, device="meta"),
                *[torch.empty_like(l) for l in logits])
    gmax = torch.stack([l.float().amax(dim=-1) for l in logits]).amax(dim=0)
    shifted = [l.float() - gmax.unsqueeze(-1) for l in logits]
    z = torch.stack([torch.exp(s).sum(dim=-1) for s in shifted]).sum(dim=0)
    nls = [-(s - torch.log(z).unsqueeze(-1)) for s in shifted]
    loss = torch.zeros_like(gmax)
    off = 0
    for nl, idx in zip(nls, indices):
        il = idx.long() - off
        ok = (il >= 0) & (il < nl.shape[-1])
        loss = loss + nl.gather(1, il.clamp(0, nl.shape[-1] - 1).unsqueeze(1)).squeeze(1) * ok.float()
        off += nl.shape[-1]
    dt = logits[0].dtype
    return (loss.to(dt), *[x.to(dt) for x in nls])


def _ce_wr_bwd_ref(*tensors, n):
    nls, indices, dloss = tensors[:n], tensors[n:2 * n], tensors[2 * n]
    if dloss.device.type == "meta":
        return tuple(torch.empty_like(x) for x in nls)
    outs, off = [], 0
    for nl, idx in zip(nls, indices):
        outs.append(_ce_bwd_ref(nl, idx.long() - off, dloss))
        off += nl.shape[-1]
    return tuple(outs)


def _vjp_ce_wr(ctx, op, gs):
    n = op.attrs["n"]
    nls = [ctx.fwd(t) for t in op.outputs[1:]]
    idx = [ctx.fwd(t) for t in op.inputs[n:]]
    return list(emit("ce_sharded_wr_grad", [*nls, *idx, gs[0]], {"n": n})) + [None] * n


OpDef("ce_sharded_wr", impl=_ce_wr_fwd_ref, vjp=_vjp_ce_wr)
OpDef("ce_sharded_wr_grad", impl=_ce_wr_bwd_ref)


def cross_entropy_sharded_wr_loss(logits: List[xl.Tensor], indices: List[xl.Tensor],
                                  ipus: Optional[Iterable[int]] = None) -> xl.Tensor:
    """Shards (possibly of different widths) are separate tensors of one replica; `indices[i]` are the original
    (un-offset) labels, one copy per shard. Returns the un-reduced loss `(n_samples,)`."""
    logits, indices = list(logits), list(indices)
    if len(logits) != len(indices):
        raise ValueError("You must provide the same number of logits and indices.")
    outs = emit("ce_sharded_wr", [*logits, *indices], {"n": len(logits)})
    return outs[0]


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
