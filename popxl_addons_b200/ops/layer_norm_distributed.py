"""LayerNorm over a hidden axis that is sharded across a replica group.

Forward: each replica sums `x` and `x^2` over its slice; one all-reduce of the `2 x N` statistics; mean and 1/std in
fp32; normalise with the local slice of gamma/beta. Backward: `sum(dy*gamma)` and `sum(dy*gamma*xhat)` are
all-reduced the same way; dgamma / dbeta are local.
Parity: popxl_addons/ops/layer_norm_distributed/layer_norm_distributed.py:21-66 (+ layer_norm_distributedx.cpp
:48-152).
"""
from typing import Optional

import torch

from .. import xl
from ..xl.opdef import OpDef, emit

__all__ = ["layer_norm_distributed"]


def _special_fwd(ex, op, env):
    group, eps = op.attrs["group"], op.attrs["eps"]
    xs, ws, bs = env[op.inputs[0]], env[op.inputs[1]], env[op.inputs[2]]
    native = ex.native_collective("layer_norm_distributed_fwd")
    if native is not None:
        res = native(ex, op, xs, ws, bs)
        if res is not NotImplemented:
            env[op.outputs[0]], env[op.outputs[1]], env[op.outputs[2]] = res
            return
    stats = [torch.stack([x.float().sum(dim=-1), (x.float() ** 2).sum(dim=-1)]) for x in xs]
    stats = ex.comm.all_reduce(stats, group, "add")
    hidden = xs[0].shape[-1] * group.group_size
    ys, means, rstds = [], [], []
    for x, w, b, s in zip(xs, ws, bs, stats):
        mean = s[0] / hidden
        var = (s[1] / hidden - mean * mean).clamp_min(0.0)
        rstd = torch.rsqrt(var + eps)
        y = (x.float() - mean.unsqueeze(-1)) * rstd.unsqueeze(-1) * w.float() + b.float()
        ys.append(y.to(x.dtype)), means.append(mean), rstds.append(rstd)
    env[op.outputs[0]], env[op.outputs[1]], env[op.outputs[2]] = ys, means, rstds


def _special_bwd(ex, op, env):
    group = op.attrs["group"]
    xs, ws, means, rstds, gs = (env[t] for t in op.inputs)
    native = ex.native_collective("layer_norm_distributed_bwd")
    if native is not None:
        res = native(ex, op, xs, ws, means, rstds, gs)
        if res is not NotImplemented:
            env[op.outputs[0]], env[op.outputs[1]], env[op.outputs[2]] = res
            return
    hidden = xs[0].shape[-1] * group.group_size
    xhats, gws, stats = [], [], []
    for x, w, m, r, g in zip(xs, ws, means, rstds, gs):
        xh = (x.float() - m.unsqueeze(-1)) * r.unsqueeze(-1)
        gw = g.float() * w.float()
        xhats.append(xh), gws.append(gw)
        stats.append(torch.stack([gw.sum(dim=-1), (gw * xh).sum(dim=-1)]))
    stats = ex.comm.all_reduce(stats, group, "add")
    dxs, dws, dbs = [], [], []
    for x, w, r, g, xh, gw, s in zip(xs, ws, rstds, gs, xhats, gws, stats):
        c1, c2 = (s[0] / hidden).unsqueeze(-1), (s[1] / hidden).unsqueeze(-1)
        dxs.append(((gw - c1 - xh * c2) * r.unsqueeze(-1)).to(x.dtype))
        dws.append((g.float() * xh).sum(dim=0).to(w.dtype))
        dbs.append(g.float().sum(dim=0).to(w.dtype))
    env[op.outputs[0]], env[op.outputs[1]], env[op.outputs[2]] = dxs, dws, dbs


def _vjp(ctx, op, gs):
    x, w, b = op.inputs
    y, mean, rstd = op.outputs
    return list(emit("layer_norm_distributed_grad",
                     [ctx.fwd(x), ctx.fwd(w), ctx.fwd(mean), ctx.fwd(rstd), gs[0]], {"group": op.attrs["group"]}))


OpDef("layer_norm_distributed", special=_special_fwd, vjp=_vjp, collective=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, ()),
                        ((op.inputs[0].shape[0],), xl.float32, ()), ((op.inputs[0].shape[0],), xl.float32, ())])
OpDef("layer_norm_distributed_grad", special=_special_bwd, collective=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, ()), (op.inputs[1].shape, op.inputs[1].dtype, ()),
                        (op.inputs[1].shape, op.inputs[1].dtype, ())])


def layer_norm_distributed(t: xl.Tensor, w: xl.Tensor, b: xl.Tensor, epsilon: float = 1e-5,
                           group: Optional[xl.ReplicaGrouping] = None) -> xl.Tensor:
    """`t (N, H/g)`, `w`/`b (H/g,)`: this replica's slice of the hidden axis and of the affine parameters."""
    if t.rank != 2 or w.rank != 1 or b.rank != 1:
        raise ValueError(f"Expected t of rank 2 and w, b of rank 1; got {t.shape}, {w.shape}, {b.shape}")
    group = group if group is not None else xl.gcg().ir.replica_grouping()
    return emit("layer_norm_distributed", [t, w, b], {"eps": float(epsilon), "group": group},
                ["outputs", "mean", "std"])[0]


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
