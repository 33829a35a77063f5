"""Operator library of the graph substrate (`xl.ops.*`).

Each function records one op in the graph being built. The torch reference implementation registered with it is
what the CPU backend runs and what every CUDA kernel is tested against; native sm_100a kernels attach themselves to
the same `OpDef` (see `popxl_addons_b200.ops.native`). The list covers the `popxl.ops` names used by popxl_addons and
its tests (layers/*.py, optimizers/adam.py:85-111, transforms/*.py, ops/cross_entropy.py:10-66).
"""
import builtins as _builtins
import math
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn.functional as F

from .. import core
from ..core import Constant, Graph, Tensor, TensorSpec, constant, gcg
from ..dtypes import dtype as _dtype
from .. import dtypes as _dt
from ..opdef import OPS, OpDef, emit, emit1, register

builtins_slice = _builtins.slice
builtins_max = _builtins.max
builtins_min = _builtins.min
builtins_sum = _builtins.sum
builtins_abs = _builtins.abs

# ===============================================================================================================
# helpers
# ===============================================================================================================


def _unbroadcast(g: Tensor, shape: Tuple[int, ...]) -> Tensor:
    """Reduce a gradient of a broadcast result back to the operand's shape."""
    if tuple(g.shape) == tuple(shape):
        return g
    gs = list(g.shape)
    lead = len(gs) - len(shape)
    axes = list(range(lead))
    for i, s in enumerate(shape):
        if s == 1 and gs[lead + i] != 1:
            axes.append(lead + i)
    if axes:
        g = sum(g, axis=axes, keepdims=False)
    if tuple(g.shape) != tuple(shape):
        g = reshape(g, shape)
    return g


def _axes(axis, rank) -> Optional[List[int]]:
    if axis is None:
        return None
    if isinstance(axis, int):
        axis = [axis]
    return [a % rank if rank else 0 for a in axis]


def _const_like(value, t: Tensor) -> Tensor:
    return constant(value, t.dtype)


# ===============================================================================================================
# elementwise binary
# ===============================================================================================================


def _vjp_add(ctx, op, gs):
    (g,) = gs
    return [_unbroadcast(g, op.inputs[0].shape), _unbroadcast(g, op.inputs[1].shape)]


def _vjp_sub(ctx, op, gs):
    (g,) = gs
    return [_unbroadcast(g, op.inputs[0].shape), _unbroadcast(negate(g), op.inputs[1].shape)]


def _vjp_mul(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    return [_unbroadcast(mul(g, ctx.fwd(b)), a.shape), _unbroadcast(mul(g, ctx.fwd(a)), b.shape)]


def _vjp_div(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    fb = ctx.fwd(b)
    ga = div(g, fb)
    gb = negate(div(mul(g, ctx.fwd(op.outputs[0])), fb))
    return [_unbroadcast(ga, a.shape), _unbroadcast(gb, b.shape)]


_WIDE_UNSIGNED = (torch.uint16, torch.uint32, torch.uint64)


def _uint_safe(fn):
    """torch has no arithmetic for 16/32/64-bit unsigned tensors: compute such operands in int64 and cast back (wraps
    modulo 2^n like the unsigned type)."""

    def f(a, b):
        if a.dtype in _WIDE_UNSIGNED or b.dtype in _WIDE_UNSIGNED:
            dt = a.dtype if a.dtype in _WIDE_UNSIGNED else b.dtype
            if a.device.type == "meta":
                return torch.empty(torch.broadcast_shapes(a.shape, b.shape), dtype=dt, device="meta")
            return fn(a.to(torch.int64), b.to(torch.int64)).to(dt)
        return fn(a, b)

    return f


register("add", vjp=_vjp_add, keeps_meta=True)(_uint_safe(torch.add))
register("sub", vjp=_vjp_sub, keeps_meta=True)(_uint_safe(torch.sub))
register("mul", vjp=_vjp_mul, keeps_meta=True)(_uint_safe(torch.mul))


def _div_ref(a, b):
    # integer operands divide like C (truncation), floats divide exactly
    if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
        return torch.div(a, b, rounding_mode="trunc")
    return torch.div(a, b)


register("div", vjp=_vjp_div, keeps_meta=True)(_div_ref)
register("fmod", keeps_meta=True)(lambda a, b: torch.fmod(a, b))
register("remainder", keeps_meta=True)(lambda a, b: torch.remainder(a, b))


def _vjp_pow(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    fa, fb, fy = ctx.fwd(a), ctx.fwd(b), ctx.fwd(op.outputs[0])
    ga = mul(g, mul(fb, div(fy, fa)))
    gb = mul(g, mul(fy, log(fa)))
    return [_unbroadcast(ga, a.shape), _unbroadcast(gb, b.shape)]


register("pow", vjp=_vjp_pow, keeps_meta=True)(lambda a, b: torch.pow(a, b))


def _vjp_maximum(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    mask = cast(greater_equal(ctx.fwd(a), ctx.fwd(b)), g.dtype)
    return [_unbroadcast(mul(g, mask), a.shape), _unbroadcast(mul(g, sub(_const_like(1, g), mask)), b.shape)]


def _vjp_minimum(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    mask = cast(less_equal(ctx.fwd(a), ctx.fwd(b)), g.dtype)
    return [_unbroadcast(mul(g, mask), a.shape), _unbroadcast(mul(g, sub(_const_like(1, g), mask)), b.shape)]


register("maximum", vjp=_vjp_maximum, keeps_meta=True)(lambda a, b: torch.maximum(a, b))
register("minimum", vjp=_vjp_minimum, keeps_meta=True)(lambda a, b: torch.minimum(a, b))
register("equal")(lambda a, b: torch.eq(a, b))
register("not_equal")(lambda a, b: torch.ne(a, b))
register("greater")(lambda a, b: torch.gt(a, b))
register("greater_equal")(lambda a, b: torch.ge(a, b))
register("less")(lambda a, b: torch.lt(a, b))
register("less_equal")(lambda a, b: torch.le(a, b))
register("logical_and")(lambda a, b: torch.logical_and(a, b))
register("logical_or")(lambda a, b: torch.logical_or(a, b))
register("logical_not")(lambda a: torch.logical_not(a))


def _bin(name):
    def f(a: Tensor, b) -> Tensor:
        if not isinstance(a, Tensor):
            a = b._lift(a)
        b = a._lift(b)
        return emit1(name, [a, b])

    f.__name__ = name
    return f


add = _bin("add")
sub = _bin("sub")
mul = _bin("mul")
div = _bin("div")
fmod = _bin("fmod")
remainder = _bin("remainder")
pow = _bin("pow")
maximum = _bin("maximum")
minimum = _bin("minimum")
equal = _bin("equal")
not_equal = _bin("not_equal")
greater = _bin("greater")
greater_equal = _bin("greater_equal")
less = _bin("less")
less_equal = _bin("less_equal")
logical_and = _bin("logical_and")
logical_or = _bin("logical_or")


def logical_not(a: Tensor) -> Tensor:
    return emit1("logical_not", [a])


# ===============================================================================================================
# elementwise unary
# ===============================================================================================================


def _unary(name, fn, vjp=None):
    OpDef(name, impl=fn, vjp=vjp, keeps_meta=True)

    def f(t: Tensor) -> Tensor:
        return emit1(name, [t])

    f.__name__ = name
    return f


negate = _unary("negate", lambda a: torch.neg(a), lambda ctx, op, gs: [negate(gs[0])])
exp = _unary("exp", lambda a: torch.exp(a), lambda ctx, op, gs: [mul(gs[0], ctx.fwd(op.outputs[0]))])
log = _unary("log", lambda a: torch.log(a), lambda ctx, op, gs: [div(gs[0], ctx.fwd(op.inputs[0]))])
log2 = _unary("log2", lambda a: torch.log2(a),
              lambda ctx, op, gs: [div(gs[0], mul(ctx.fwd(op.inputs[0]), _const_like(math.log(2.0), gs[0])))])
sqrt = _unary("sqrt", lambda a: torch.sqrt(a),
              lambda ctx, op, gs: [div(gs[0], mul(ctx.fwd(op.outputs[0]), _const_like(2.0, gs[0])))])
rsqrt = _unary("rsqrt", lambda a: torch.rsqrt(a),
               lambda ctx, op, gs: [mul(gs[0], mul(_const_like(-0.5, gs[0]),
                                                   div(ctx.fwd(op.outputs[0]), ctx.fwd(op.inputs[0]))))])
abs = _unary("abs", lambda a: torch.abs(a), lambda ctx, op, gs: [mul(gs[0], sign(ctx.fwd(op.inputs[0])))])
sign = _unary("sign", lambda a: torch.sign(a), lambda ctx, op, gs: [None])
floor = _unary("floor", lambda a: torch.floor(a), lambda ctx, op, gs: [None])
ceil = _unary("ceil", lambda a: torch.ceil(a), lambda ctx, op, gs: [None])
round = _unary("round", lambda a: torch.round(a), lambda ctx, op, gs: [None])
square = _unary("square", lambda a: torch.square(a),
                lambda ctx, op, gs: [mul(gs[0], mul(ctx.fwd(op.inputs[0]), _const_like(2.0, gs[0])))])
tanh = _unary("tanh", lambda a: torch.tanh(a),
              lambda ctx, op, gs: [mul(gs[0], sub(_const_like(1.0, gs[0]), square(ctx.fwd(op.outputs[0]))))])
sigmoid = _unary("sigmoid", lambda a: torch.sigmoid(a),
                 lambda ctx, op, gs: [mul(gs[0], mul(ctx.fwd(op.outputs[0]),
                                                     sub(_const_like(1.0, gs[0]), ctx.fwd(op.outputs[0]))))])
relu = _unary("relu", lambda a: torch.relu(a),
              lambda ctx, op, gs: [mul(gs[0], cast(greater(ctx.fwd(op.inputs[0]), _const_like(0, op.inputs[0])),
                                                   gs[0].dtype))])
sin = _unary("sin", lambda a: torch.sin(a), lambda ctx, op, gs: [mul(gs[0], cos(ctx.fwd(op.inputs[0])))])
cos = _unary("cos", lambda a: torch.cos(a), lambda ctx, op, gs: [negate(mul(gs[0], sin(ctx.fwd(op.inputs[0]))))])
isnan = _unary("isnan", lambda a: torch.isnan(a))
isinf = _unary("isinf", lambda a: torch.isinf(a))
detach = _unary("detach", lambda a: a.detach(), lambda ctx, op, gs: [None])
identity = _unary("identity", lambda a: a, lambda ctx, op, gs: [gs[0]])
io_tile_copy = _unary("io_tile_copy", lambda a: a, lambda ctx, op, gs: [gs[0]])
rename = identity

# ---- activations with fused backward ops ---------------------------------------------------------------------


def _gelu_ref(x, approximate="none"):
    return F.gelu(x.float(), approximate=approximate).to(x.dtype)


def _gelu_grad_ref(x, g, approximate="none"):
    xf = x.float()
    if approximate == "tanh":
        k = math.sqrt(2.0 / math.pi)
        inner = k * (xf + 0.044715 * xf ** 3)
        t = torch.tanh(inner)
        d = 0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * k * (1 + 3 * 0.044715 * xf * xf)
    else:
        cdf = 0.5 * (1.0 + torch.erf(xf * (1.0 / math.sqrt(2.0))))
        pdf = torch.exp(-0.5 * xf * xf) * (1.0 / math.sqrt(2.0 * math.pi))
        d = cdf + xf * pdf
    return (g.float() * d).to(x.dtype)


OpDef("gelu", impl=_gelu_ref, keeps_meta=True,
      vjp=lambda ctx, op, gs: [emit1("gelu_grad", [ctx.fwd(op.inputs[0]), gs[0]], dict(op.attrs))])
OpDef("gelu_grad", impl=_gelu_grad_ref, keeps_meta=True)


def gelu(t: Tensor, approximate: str = "none") -> Tensor:
    """GELU; `approximate="tanh"` selects the tanh form. On CUDA this is a hand-written vectorised kernel."""
    return emit1("gelu", [t], {"approximate": approximate})


gelu_ = gelu


def _silu_grad_ref(x, g):
    xf = x.float()
    s = torch.sigmoid(xf)
    return (g.float() * (s * (1 + xf * (1 - s)))).to(x.dtype)


OpDef("swish", impl=lambda x: F.silu(x.float()).to(x.dtype), keeps_meta=True,
      vjp=lambda ctx, op, gs: [emit1("swish_grad", [ctx.fwd(op.inputs[0]), gs[0]])])
OpDef("swish_grad", impl=_silu_grad_ref, keeps_meta=True)


def swish(t: Tensor) -> Tensor:
    return emit1("swish", [t])


silu = swish


def _swiglu_ref(gate, up):
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def _swiglu_grad_ref(gate, up, g):
    gf, uf, dy = gate.float(), up.float(), g.float()
    s = torch.sigmoid(gf)
    dgate = dy * uf * (s * (1 + gf * (1 - s)))
    dup = dy * gf * s
    return dgate.to(gate.dtype), dup.to(up.dtype)


OpDef("swiglu", impl=_swiglu_ref,
      vjp=lambda ctx, op, gs: emit("swiglu_grad", [ctx.fwd(op.inputs[0]), ctx.fwd(op.inputs[1]), gs[0]]))
OpDef("swiglu_grad", impl=_swiglu_grad_ref)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """`silu(gate) * up` in one pass (Llama FFN)."""
    return emit1("swiglu", [gate, up])


# ---- clip / cast / where -------------------------------------------------------------------------------------


def _vjp_clip(ctx, op, gs):
    x = ctx.fwd(op.inputs[0])
    lo, hi = op.attrs["min"], op.attrs["max"]
    m = logical_and(greater_equal(x, _const_like(lo, x)), less_equal(x, _const_like(hi, x)))
    return [mul(gs[0], cast(m, gs[0].dtype))]


OpDef("clip", impl=lambda a, min, max: torch.clamp(a, min, max), vjp=_vjp_clip, keeps_meta=True)


def clip(t: Tensor, min: float = -float("inf"), max: float = float("inf")) -> Tensor:
    return emit1("clip", [t], {"min": min, "max": max})


OpDef("cast", impl=lambda a, to: a.to(to.as_torch()), keeps_meta=True,
      vjp=lambda ctx, op, gs: [cast(gs[0], op.inputs[0].dtype) if op.inputs[0].dtype.is_floating_point else None])


def cast(t: Tensor, data_type: _dtype) -> Tensor:
    data_type = _dtype.as_dtype(data_type)
    if t.dtype == data_type:
        return t
    return emit1("cast", [t], {"to": data_type})


def _vjp_where(ctx, op, gs):
    c, a, b = op.inputs
    fc = ctx.fwd(c)
    z = _const_like(0, gs[0])
    return [None, _unbroadcast(where(fc, gs[0], z), a.shape), _unbroadcast(where(fc, z, gs[0]), b.shape)]


OpDef("where", impl=lambda c, a, b: torch.where(c, a, b), vjp=_vjp_where)


def where(condition: Tensor, lhs, rhs) -> Tensor:
    if not isinstance(lhs, Tensor):
        lhs = rhs._lift(lhs)
    rhs = lhs._lift(rhs)
    return emit1("where", [condition, lhs, rhs])


# ===============================================================================================================
# shape ops
# ===============================================================================================================


OpDef("reshape", impl=lambda a, shape: a.reshape(shape),
      vjp=lambda ctx, op, gs: [reshape(gs[0], op.inputs[0].shape)])


def reshape(t: Tensor, shape: Iterable[int]) -> Tensor:
    shape = tuple(int(s) for s in shape)
    if shape.count(-1) > 1:
        raise ValueError("Reshape shape can contain at most one -1")
    if -1 in shape:
        known = int(np.prod([s for s in shape if s != -1])) if len(shape) > 1 else 1
        shape = tuple(t.nelms // builtins_max(known, 1) if s == -1 else s for s in shape)
    if int(np.prod(shape)) != t.nelms and not (shape == () and t.nelms == 1):
        raise ValueError(f"Cannot reshape {t.shape} into {shape}")
    if shape == tuple(t.shape):
        return t
    return emit1("reshape", [t], {"shape": shape})


reshape_ = reshape


def flatten(t: Tensor) -> Tensor:
    return reshape(t, (-1,))


flatten_ = flatten


def squeeze(t: Tensor, axes: Optional[Iterable[int]] = None) -> Tensor:
    axes = _axes(list(axes) if axes is not None else None, t.rank)
    shape = [s for i, s in enumerate(t.shape) if not (s == 1 and (axes is None or i in axes))]
    return reshape(t, shape)


def unsqueeze(t: Tensor, axes: Iterable[int]) -> Tensor:
    shape = list(t.shape)
    for a in sorted(a % (len(shape) + 1 + i) if a < 0 else a for i, a in enumerate(axes)):
        shape.insert(a, 1)
    return reshape(t, shape)


def _vjp_transpose(ctx, op, gs):
    perm = op.attrs["perm"]
    inv = [0] * len(perm)
    for i, p in enumerate(perm):
        inv[p] = i
    return [transpose(gs[0], inv)]


OpDef("transpose", impl=lambda a, perm: a.permute(perm), vjp=_vjp_transpose)


def transpose(t: Tensor, permutation: Optional[Iterable[int]] = None) -> Tensor:
    perm = tuple(permutation) if permutation is not None else tuple(reversed(range(t.rank)))
    perm = tuple(p % t.rank for p in perm)
    if perm == tuple(range(t.rank)) and t.rank != 1:
        return t  # nothing moves: no op (a rank-1 `.T` still records one, as popxl does, so op ids line up)
    return emit1("transpose", [t], {"perm": perm})


transpose_ = transpose


def _slice_ref(a, start, stop, step, axis):
    idx = [builtins_slice(None)] * a.dim()
    for s, e, st, ax in zip(start, stop, step, axis):
        idx[ax] = builtins_slice(s, e, st)
    return a[tuple(idx)]


def _vjp_slice(ctx, op, gs):
    return [emit1("slice_grad", [gs[0]], dict(op.attrs, in_shape=tuple(op.inputs[0].shape)))]


def _slice_grad_ref(g, start, stop, step, axis, in_shape):
    out = g.new_zeros(in_shape)
    idx = [builtins_slice(None)] * len(in_shape)
    for s, e, st, ax in zip(start, stop, step, axis):
        idx[ax] = builtins_slice(s, e, st)
    out[tuple(idx)] = g
    return out


OpDef("slice", impl=_slice_ref, vjp=_vjp_slice)
OpDef("slice_grad", impl=_slice_grad_ref)


def slice(t: Tensor, start=None, stop=None, step=None, axis=None) -> Tensor:
    def listify(v):
        return [v] if isinstance(v, int) else (list(v) if v is not None else None)

    start, stop, step, axis = listify(start), listify(stop), listify(step), listify(axis)
    n = builtins_max(len(v) for v in (start, stop, step, axis) if v is not None)
    axis = axis if axis is not None else list(range(n))
    axis = [a % t.rank for a in axis]
    start = start if start is not None else [0] * n
    stop = stop if stop is not None else [t.shape[a] for a in axis]
    step = step if step is not None else [1] * n
    return emit1("slice", [t], {"start": tuple(start), "stop": tuple(stop), "step": tuple(step), "axis": tuple(axis)})


slice_ = slice


def subscript(t: Tensor, key) -> Tensor:
    """`t[key]` for ints, slices, None and Ellipsis (static indices only)."""
    if not isinstance(key, tuple):
        key = (key,)
    if any(k is Ellipsis for k in key):
        i = [n for n, k in enumerate(key) if k is Ellipsis][0]
        n_real = len([k for k in key if k is not None and k is not Ellipsis])
        key = key[:i] + (builtins_slice(None),) * (t.rank - n_real) + key[i + 1:]
    starts, stops, steps, axes, squeeze_axes, new_axes = [], [], [], [], [], []
    ax = 0
    out_pos = 0
    for k in key:
        if k is None:
            new_axes.append(out_pos)
            out_pos += 1
            continue
        if isinstance(k, int):
            k = k % t.shape[ax]
            starts.append(k), stops.append(k + 1), steps.append(1), axes.append(ax)
            squeeze_axes.append(ax)
            ax += 1
            continue
        if isinstance(k, builtins_slice):
            s, e, st = k.indices(t.shape[ax])
            if (s, e, st) != (0, t.shape[ax], 1):
                starts.append(s), stops.append(e), steps.append(st), axes.append(ax)
            ax += 1
            out_pos += 1
            continue
        raise TypeError(f"Unsupported index {k!r}")
    out = slice(t, starts, stops, steps, axes) if axes else t
    if squeeze_axes:
        out = reshape(out, [s for i, s in enumerate(out.shape) if i not in squeeze_axes])
    if new_axes:
        out = unsqueeze(out, new_axes)
    return out




def _vjp_concat(ctx, op, gs):
    axis = op.attrs["axis"]
    out, off = [], 0
    for t in op.inputs:
        out.append(slice(gs[0], [off], [off + t.shape[axis]], [1], [axis]))
        off += t.shape[axis]
    return out


OpDef("concat", impl=lambda *ts, axis: torch.cat(ts, dim=axis), vjp=_vjp_concat)


def concat(ts: Iterable[Tensor], axis: int = 0) -> Tensor:
    ts = list(ts)
    if len(ts) == 1:
        return ts[0]
    return emit1("concat", ts, {"axis": axis % ts[0].rank})


concat_ = concat


def split(t: Tensor, splits: Union[int, List[int]], axis: int = 0) -> List[Tensor]:
    axis = axis % t.rank
    if isinstance(splits, int):
        assert t.shape[axis] % splits == 0
        splits = [t.shape[axis] // splits] * splits
    out, off = [], 0
    for s in splits:
        out.append(slice(t, [off], [off + s], [1], [axis]))
        off += s
    return out


def _vjp_expand(ctx, op, gs):
    return [_unbroadcast(gs[0], op.inputs[0].shape)]


OpDef("expand", impl=lambda a, shape: a.expand(shape), vjp=_vjp_expand)


def expand(t: Tensor, shape: Iterable[int]) -> Tensor:
    return emit1("expand", [t], {"shape": tuple(shape)})


def _vjp_tile(ctx, op, gs):
    """Gradient of `tile`: every element of the operand appears `prod(repeats)` times in the result, so its gradient is
    the sum over the copies. The result is viewed as (r0, s0, r1, s1, ...) and the repeat axes are summed."""
    x = op.inputs[0]
    reps = tuple(op.attrs["repeats"])
    shape = (1,) * (len(reps) - x.rank) + tuple(x.shape)
    split = []
    for r, n in zip(reps, shape):
        split += [r, n]
    g = reshape(gs[0], tuple(split))
    g = sum(g, axis=list(range(0, 2 * len(reps), 2)), keepdims=False)
    return [reshape(g, tuple(x.shape))]


OpDef("tile", impl=lambda a, repeats: a.repeat(repeats), vjp=_vjp_tile)


def tile(t: Tensor, repeats: Iterable[int]) -> Tensor:
    return emit1("tile", [t], {"repeats": tuple(repeats)})


# ===============================================================================================================
# reductions
# ===============================================================================================================


def _red_ref(fn):
    def f(a, axis, keepdims):
        if axis is None:
            axis = list(range(a.dim()))
        if len(axis) == 0:
            return a.clone()
        return fn(a, axis, keepdims)

    return f


def _expand_grad(op, g):
    """Reshape/broadcast the gradient of a reduction back to the reduced operand's shape."""
    x = op.inputs[0]
    axis = op.attrs["axis"] if op.attrs["axis"] is not None else list(range(x.rank))
    if not op.attrs["keepdims"]:
        shape = [1 if i in axis else s for i, s in enumerate(x.shape)]
        g = reshape(g, shape)
    return expand(g, x.shape)


def _vjp_sum(ctx, op, gs):
    return [_expand_grad(op, gs[0])]


def _vjp_mean(ctx, op, gs):
    x = op.inputs[0]
    n = x.nelms // builtins_max(op.outputs[0].nelms, 1)
    return [div(_expand_grad(op, gs[0]), _const_like(float(n), gs[0]))]


def _vjp_max(ctx, op, gs):
    x = op.inputs[0]
    y = _expand_grad(op, ctx.fwd(op.outputs[0]))
    mask = cast(equal(ctx.fwd(x), y), gs[0].dtype)
    return [mul(_expand_grad(op, gs[0]), mask)]


OpDef("sum", impl=_red_ref(lambda a, ax, k: torch.sum(a, dim=ax, keepdim=k)), vjp=_vjp_sum)
OpDef("mean", impl=_red_ref(lambda a, ax, k: torch.mean(a, dim=ax, keepdim=k)), vjp=_vjp_mean)
OpDef("max", impl=_red_ref(lambda a, ax, k: torch.amax(a, dim=ax, keepdim=k)), vjp=_vjp_max)
OpDef("min", impl=_red_ref(lambda a, ax, k: torch.amin(a, dim=ax, keepdim=k)), vjp=_vjp_max)
OpDef("prod", impl=_red_ref(lambda a, ax, k: torch.prod(a, dim=ax[0], keepdim=k)))
OpDef("sumsquare", impl=_red_ref(lambda a, ax, k: torch.sum(a * a, dim=ax, keepdim=k)))
OpDef("l2", impl=_red_ref(lambda a, ax, k: torch.sqrt(torch.sum(a * a, dim=ax, keepdim=k))))
OpDef("l1", impl=_red_ref(lambda a, ax, k: torch.sum(a.abs(), dim=ax, keepdim=k)))


def _reduce(name):
    def f(t: Tensor, axis: Optional[Union[int, Iterable[int]]] = None, keepdims: bool = False) -> Tensor:
        ax = _axes(axis, t.rank)
        return emit1(name, [t], {"axis": ax, "keepdims": bool(keepdims)})

    f.__name__ = name
    return f


sum = _reduce("sum")
mean = _reduce("mean")
max = _reduce("max")
min = _reduce("min")
prod = _reduce("prod")
sumsquare = _reduce("sumsquare")
l2 = _reduce("l2")
l1 = _reduce("l1")

OpDef("argmax", impl=lambda a, dim, keepdim: torch.argmax(a, dim=dim, keepdim=keepdim).to(torch.int32))
OpDef("argmin", impl=lambda a, dim, keepdim: torch.argmin(a, dim=dim, keepdim=keepdim).to(torch.int32))


def argmax(t: Tensor, dim: int = 0, keepdim: bool = False) -> Tensor:
    return emit1("argmax", [t], {"dim": dim, "keepdim": keepdim})


def argmin(t: Tensor, dim: int = 0, keepdim: bool = False) -> Tensor:
    return emit1("argmin", [t], {"dim": dim, "keepdim": keepdim})


OpDef("cumsum", impl=lambda a, dim: torch.cumsum(a, dim=dim),
      vjp=lambda ctx, op, gs: [emit1("cumsum_rev", [gs[0]], dict(op.attrs))])
OpDef("cumsum_rev", impl=lambda a, dim: torch.flip(torch.cumsum(torch.flip(a, [dim]), dim=dim), [dim]))


def cumsum(t: Tensor, dim: int = 0) -> Tensor:
    return emit1("cumsum", [t], {"dim": dim % t.rank})


def _topk_ref(a, k, axis, largest, sorted):
    v, i = torch.topk(a, k, dim=axis, largest=largest, sorted=sorted)
    return v, i.to(torch.int32)


OpDef("topk", impl=_topk_ref)


def topk(t: Tensor, k: int, axis: int = -1, largest: bool = True, sorted: bool = True):
    v, i = emit("topk", [t], {"k": k, "axis": axis, "largest": largest, "sorted": sorted})
    return v, i


# ===============================================================================================================
# matmul / softmax / normalisation / gather
# ===============================================================================================================


def _matmul_ref(a, b):
    if a.dtype != b.dtype:
        b = b.to(a.dtype)
    return torch.matmul(a, b)


def _vjp_matmul(ctx, op, gs):
    (g,) = gs
    a, b = op.inputs
    fa, fb = ctx.fwd(a), ctx.fwd(b)

    def t_last(x):
        if x.rank < 2:
            return x
        perm = list(range(x.rank))
        perm[-1], perm[-2] = perm[-2], perm[-1]
        return transpose(x, perm)

    if a.rank == 1 and b.rank == 1:
        return [mul(g, fb), mul(g, fa)]
    if a.rank == 1:
        if b.rank != 2:
            raise NotImplementedError("matmul vjp for 1-D x N-D")
        return [matmul(fb, g), matmul(reshape(fa, (-1, 1)), reshape(g, (1, -1)))]
    if b.rank == 1:
        ga = matmul(reshape(g, (*g.shape, 1)), reshape(fb, (1, -1)))
        gb = matmul(reshape(g, (1, -1)), reshape(fa, (-1, a.shape[-1])))
        return [ga, reshape(gb, b.shape)]
    ga = matmul(g, t_last(fb))
    # weight gradient: collapse leading (batch) dims of a 2-D weight into one GEMM
    if b.rank == 2 and a.rank > 2:
        gb = matmul(transpose(reshape(fa, (-1, a.shape[-1]))), reshape(g, (-1, g.shape[-1])))
    else:
        gb = matmul(t_last(fa), g)
    return [_unbroadcast(ga, a.shape), _unbroadcast(gb, b.shape)]


def _matmul_flops(op):
    a, b = op.inputs
    k = a.shape[-1]
    return 2 * k * op.outputs[0].nelms


OpDef("matmul", impl=_matmul_ref, vjp=_vjp_matmul, flops=_matmul_flops)


def matmul(lhs: Tensor, rhs: Tensor, available_memory_proportion=None, output_type=None,
           partials_type=None) -> Tensor:
    """`lhs @ rhs` with numpy broadcasting rules. The planner hints are accepted and recorded only."""
    outs = emit("matmul", [lhs, rhs])
    if available_memory_proportion is not None:
        outs[0].producer.attrs_hint = available_memory_proportion
    return outs[0]


def _vjp_softmax(ctx, op, gs):
    y = ctx.fwd(op.outputs[0])
    return [emit1("softmax_grad", [y, gs[0]], dict(op.attrs))]


def _softmax_grad_ref(y, g, axis):
    yf, gf = y.float(), g.float()
    return (yf * (gf - (gf * yf).sum(dim=axis, keepdim=True))).to(y.dtype)


OpDef("softmax", impl=lambda a, axis: torch.softmax(a.float(), dim=axis).to(a.dtype), vjp=_vjp_softmax)
OpDef("softmax_grad", impl=_softmax_grad_ref)
OpDef("logsoftmax", impl=lambda a, axis: torch.log_softmax(a.float(), dim=axis).to(a.dtype),
      vjp=lambda ctx, op, gs: [sub(gs[0], mul(exp(ctx.fwd(op.outputs[0])),
                                              sum(gs[0], axis=op.attrs["axis"], keepdims=True)))])


def softmax(t: Tensor, axis: int = -1) -> Tensor:
    return emit1("softmax", [t], {"axis": axis % t.rank})


def logsoftmax(t: Tensor, axis: int = -1) -> Tensor:
    return emit1("logsoftmax", [t], {"axis": axis % t.rank})


# ---- layer norm / rms norm / group norm (fused fwd saves mean & rstd; fused bwd) -----------------------------


def _ln_fwd_ref(x, w, b, eps):
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean) * rstd * w.float() + b.float()
    return y.to(x.dtype), mean.squeeze(-1), rstd.squeeze(-1)


def _ln_bwd_ref(x, w, mean, rstd, g):
    xf, gf, wf = x.float(), g.float(), w.float()
    xhat = (xf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
    gw = gf * wf
    c1 = gw.mean(dim=-1, keepdim=True)
    c2 = (gw * xhat).mean(dim=-1, keepdim=True)
    dx = (gw - c1 - xhat * c2) * rstd.unsqueeze(-1)
    red = tuple(range(x.dim() - 1))
    dw = (gf * xhat).sum(dim=red)
    db = gf.sum(dim=red)
    return dx.to(x.dtype), dw.to(w.dtype), db.to(w.dtype)


def _vjp_ln(ctx, op, gs):
    x, w, b = op.inputs
    y, mean, rstd = op.outputs
    dx, dw, db = emit("layer_norm_grad", [ctx.fwd(x), ctx.fwd(w), ctx.fwd(mean), ctx.fwd(rstd), gs[0]])
    return [dx, dw, db]


OpDef("layer_norm", impl=_ln_fwd_ref, vjp=_vjp_ln)
OpDef("layer_norm_grad", impl=_ln_bwd_ref)


def layer_norm(t: Tensor, weight: Tensor, bias: Tensor, eps: float = 1e-5) -> Tensor:
    """LayerNorm over the last axis. One fused kernel forward (saves mean and 1/std), one fused kernel backward."""
    return emit("layer_norm", [t, weight, bias], {"eps": float(eps)})[0]


def _rms_fwd_ref(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype), rstd.squeeze(-1)


def _rms_bwd_ref(x, w, rstd, g):
    xf, gf, wf = x.float(), g.float(), w.float()
    r = rstd.unsqueeze(-1)
    xhat = xf * r
    gw = gf * wf
    c = (gw * xhat).mean(dim=-1, keepdim=True)
    dx = (gw - xhat * c) * r
    dw = (gf * xhat).sum(dim=tuple(range(x.dim() - 1)))
    return dx.to(x.dtype), dw.to(w.dtype)


OpDef("rms_norm", impl=_rms_fwd_ref,
      vjp=lambda ctx, op, gs: emit("rms_norm_grad", [ctx.fwd(op.inputs[0]), ctx.fwd(op.inputs[1]),
                                                     ctx.fwd(op.outputs[1]), gs[0]]))
OpDef("rms_norm_grad", impl=_rms_bwd_ref)


def rms_norm(t: Tensor, weight: Tensor, eps: float = 1e-5) -> Tensor:
    return emit("rms_norm", [t, weight], {"eps": float(eps)})[0]


def _gn_ref(x, w, b, num_groups, eps):
    return F.group_norm(x.float(), num_groups, w.float(), b.float(), eps).to(x.dtype)


def _gn_grad_ref(x, w, b, g, num_groups, eps):
    with torch.enable_grad():
        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().float().requires_grad_(True)
        br = b.detach().float().requires_grad_(True)
        y = F.group_norm(xr, num_groups, wr, br, eps)
        dx, dw, db = torch.autograd.grad(y, (xr, wr, br), g.float())
    return dx.to(x.dtype), dw.to(w.dtype), db.to(b.dtype)


def _infer_like_inputs(n):
    def infer(op):
        return [(t.shape, t.dtype, ()) for t in op.inputs[:n]]

    return infer


OpDef("group_norm", impl=_gn_ref,
      vjp=lambda ctx, op, gs: emit("group_norm_grad", [ctx.fwd(op.inputs[0]), ctx.fwd(op.inputs[1]),
                                                       ctx.fwd(op.inputs[2]), gs[0]], dict(op.attrs)))
OpDef("group_norm_grad", impl=_gn_grad_ref, infer=_infer_like_inputs(3))


def group_norm(t: Tensor, weight: Tensor, bias: Tensor, num_groups: int, eps: float = 1e-5) -> Tensor:
    return emit1("group_norm", [t, weight, bias], {"num_groups": int(num_groups), "eps": float(eps)})


# ---- conv ----------------------------------------------------------------------------------------------------


def _conv_ref(x, w, stride, padding, dilation, groups):
    pl = list(padding)
    # padding = (top, left, bottom, right) explicit
    xt = F.pad(x, (pl[1], pl[3], pl[0], pl[2])) if any(pl) else x
    return F.conv2d(xt, w.to(x.dtype), None, stride, 0, dilation, groups)


def _conv_grad_ref(x, w, g, stride, padding, dilation, groups):
    with torch.enable_grad():
        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().float().requires_grad_(True)
        y = _conv_ref(xr, wr, stride, padding, dilation, groups)
        dx, dw = torch.autograd.grad(y, (xr, wr), g.float())
    return dx.to(x.dtype), dw.to(w.dtype)


OpDef("conv", impl=_conv_ref,
      vjp=lambda ctx, op, gs: emit("conv_grad", [ctx.fwd(op.inputs[0]), ctx.fwd(op.inputs[1]), gs[0]],
                                   dict(op.attrs)))
OpDef("conv_grad", impl=_conv_grad_ref, infer=_infer_like_inputs(2))


def conv(t: Tensor, weight: Tensor, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), groups: int = 1,
         pad_type: str = "not_set", available_memory_proportions=None, partials_types=None,
         enable_conv_dithering=None, output_type=None, cycle_back_off=None, available_memory_proportion=None,
         partials_type=None) -> Tensor:
    """2-D convolution, NCHW. `padding` is explicit `(top, left, bottom, right)`; `pad_type` may be
    `same_upper`, `same_lower` or `valid` to derive it. Planner knobs are accepted for API parity and ignored."""
    stride, dilation = tuple(stride), tuple(dilation)
    padding = tuple(padding)
    if pad_type in ("same_upper", "same_lower"):
        pads = []
        for i in range(2):
            in_sz, k = t.shape[2 + i], weight.shape[2 + i]
            out_sz = -(-in_sz // stride[i])
            total = builtins_max((out_sz - 1) * stride[i] + (k - 1) * dilation[i] + 1 - in_sz, 0)
            lo, hi = total // 2, total - total // 2
            pads.append((lo, hi) if pad_type == "same_upper" else (hi, lo))
        padding = (pads[0][0], pads[1][0], pads[0][1], pads[1][1])
    elif pad_type == "valid":
        padding = (0, 0, 0, 0)
    return emit1("conv", [t, weight], {"stride": stride, "padding": padding, "dilation": dilation,
                                       "groups": int(groups)})


# ---- gather / scatter ----------------------------------------------------------------------------------------


def _gather_ref(w, idx, axis, zero_OOR):
    idx_l = idx.long()
    n = w.shape[axis]
    if zero_OOR:
        oor = (idx_l < 0) | (idx_l >= n)
        safe = idx_l.clamp(0, n - 1)
    else:
        safe = idx_l
    out = torch.index_select(w, axis, safe.reshape(-1))
    out = out.reshape(*w.shape[:axis], *idx.shape, *w.shape[axis + 1:])
    if zero_OOR:
        mask_shape = [1] * axis + list(idx.shape) + [1] * (w.dim() - axis - 1)
        out = out * (~oor).reshape(mask_shape).to(out.dtype)
    return out


def _gather_grad_ref(g, idx, axis, zero_OOR, w_shape):
    out = g.new_zeros(w_shape, dtype=torch.float32)
    idx_l = idx.long().reshape(-1)
    n = w_shape[axis]
    gf = g.float().reshape(*w_shape[:axis], -1, *w_shape[axis + 1:])
    valid = (idx_l >= 0) & (idx_l < n)
    gf = gf * valid.reshape([1] * axis + [-1] + [1] * (len(w_shape) - axis - 1)).to(gf.dtype)
    out.index_add_(axis, idx_l.clamp(0, n - 1), gf)
    return out.to(g.dtype)


OpDef("gather", impl=_gather_ref,
      vjp=lambda ctx, op, gs: [emit1("gather_grad", [gs[0], ctx.fwd(op.inputs[1])],
                                     dict(op.attrs, w_shape=tuple(op.inputs[0].shape))), None])
OpDef("gather_grad", impl=_gather_grad_ref)


def gather(t: Tensor, indices: Tensor, axis: int = 0, available_memory_proportion=None,
           zero_OOR: bool = False) -> Tensor:
    """Select slices of `t` along `axis`. With `zero_OOR` out-of-range indices yield zeros (vocab-sharded lookup)."""
    return emit1("gather", [t, indices], {"axis": axis % t.rank, "zero_OOR": bool(zero_OOR)})


def _onehot_ref(idx, num_classes, dt):
    return F.one_hot(idx.long(), num_classes).to(dt.as_torch())


OpDef("onehot", impl=_onehot_ref)


def onehot(t: Tensor, num_classes: int, values=None, axis: int = -1, dtype=None) -> Tensor:
    return emit1("onehot", [t], {"num_classes": int(num_classes), "dt": _dtype.as_dtype(dtype or _dt.float32)})


# ---- dynamic slice / update (stash ring buffers) -------------------------------------------------------------


def _dyn_positions(index, size):
    """`index + [0, size)` as an int64 vector on the index's device: the slice is taken on the device, so a stash ring
    inside a captured loop needs no host read."""
    return index.reshape(-1)[:1].to(torch.int64) + torch.arange(size, device=index.device)


def _dyn_slice_ref(t, index, axes, sizes):
    assert len(axes) == 1
    if index.device.type == "meta":
        return t.narrow(axes[0], 0, sizes[0]).clone()
    if index.device.type == "cpu":
        i = int(index.reshape(-1)[0])
        return t.narrow(axes[0], i, sizes[0]).clone()
    pos = _dyn_positions(index, sizes[0]).clamp(0, t.shape[axes[0]] - 1)
    return t.index_select(axes[0], pos)


def _dyn_update_ref(t, index, update, axes, sizes):
    if t.device.type == "meta":
        return t
    if index.device.type == "cpu":
        i = int(index.reshape(-1)[0])
        t.narrow(axes[0], i, sizes[0]).copy_(update)
        return t
    pos = _dyn_positions(index, sizes[0]).clamp(0, t.shape[axes[0]] - 1)
    t.index_copy_(axes[0], pos, update.reshape(*t.shape[:axes[0]], sizes[0], *t.shape[axes[0] + 1:]))
    return t


OpDef("dynamic_slice", impl=_dyn_slice_ref)
OpDef("dynamic_update_", impl=_dyn_update_ref, inplace=True)


def dynamic_slice(t: Tensor, index: Tensor, axes: List[int], sizes: List[int], no_overlap: bool = True) -> Tensor:
    return emit1("dynamic_slice", [t, index], {"axes": tuple(axes), "sizes": tuple(sizes)})


def dynamic_update_(t: Tensor, index: Tensor, update: Tensor, axes: List[int], sizes: List[int],
                    no_overlap: bool = True) -> Tensor:
    return emit1("dynamic_update_", [t, index, update], {"axes": tuple(axes), "sizes": tuple(sizes)})


dynamic_update = dynamic_update_


def _incmod_ref(t, increment, modulus):
    if t.device.type == "meta":
        return t
    v = t.view(torch.int32) if t.dtype == torch.uint32 else t
    v.add_(int(increment) if not t.dtype.is_floating_point else increment)
    v.remainder_(int(modulus) if not t.dtype.is_floating_point else modulus)
    return t


OpDef("increment_mod_", impl=_incmod_ref, inplace=True)
OpDef("increment_mod", impl=lambda t, increment, modulus: _incmod_ref(t.clone(), increment, modulus))


def increment_mod_(t: Tensor, increment: float, modulus: float) -> Tensor:
    return emit1("increment_mod_", [t], {"increment": increment, "modulus": modulus})


def increment_mod(t: Tensor, increment: float, modulus: float) -> Tensor:
    return emit1("increment_mod", [t], {"increment": increment, "modulus": modulus})


# ===============================================================================================================
# in-place arithmetic
# ===============================================================================================================


def _add_inplace_ref(a, b):
    if a.device.type == "meta":
        return a
    return a.add_(b.to(a.dtype))


OpDef("add_", impl=_add_inplace_ref, inplace=True, keeps_meta=True)


def add_(lhs: Tensor, rhs) -> Tensor:
    return emit1("add_", [lhs, lhs._lift(rhs)])


def _copy_inplace_ref(dst, src):
    if dst.device.type == "meta":
        return dst
    return dst.copy_(src)


OpDef("copy_var_update_", impl=_copy_inplace_ref, inplace=True, keeps_meta=True)


def _scaled_add_ref(x, y, *scalars, a, b, has_a, has_b, inplace):
    it = iter(scalars)
    av = next(it) if has_a else a
    bv = next(it) if has_b else b
    if x.device.type == "meta":
        return x if inplace else torch.empty_like(x)
    av = av.to(torch.float32) if isinstance(av, torch.Tensor) else av
    bv = bv.to(torch.float32) if isinstance(bv, torch.Tensor) else bv
    res = (x.float() * av + y.float() * bv).to(x.dtype)
    if inplace:
        return x.copy_(res)
    return res


OpDef("scaled_add", impl=_scaled_add_ref, keeps_meta=True)
OpDef("scaled_add_", impl=_scaled_add_ref, inplace=True, keeps_meta=True)


def _scaled_add(name, X, Y, a, b, inplace):
    ins = [X, Y]
    has_a, has_b = isinstance(a, Tensor), isinstance(b, Tensor)
    if has_a:
        ins.append(a)
    if has_b:
        ins.append(b)
    return emit1(name, ins, {"a": None if has_a else float(a), "b": None if has_b else float(b),
                             "has_a": has_a, "has_b": has_b, "inplace": inplace})


def scaled_add(X: Tensor, Y: Tensor, a=1.0, b=1.0) -> Tensor:
    """`a*X + b*Y`; `a`, `b` may be floats or scalar tensors."""
    return _scaled_add("scaled_add", X, Y, a, b, False)


def scaled_add_(X: Tensor, Y: Tensor, a=1.0, b=1.0) -> Tensor:
    """In-place `X = a*X + b*Y`."""
    return _scaled_add("scaled_add_", X, Y, a, b, True)


# ===============================================================================================================
# init / random
# ===============================================================================================================


def _infer_init(op):
    return [(op.attrs["shape"], op.attrs["dt"], op.attrs.get("meta_shape", ()))]


def _special_init(ex, op, env):
    shape, dt = op.attrs["shape"], op.attrs["dt"].as_torch()
    vals = []
    for r in range(ex.num_local):
        if op.attrs["init_type"] == "zero":
            vals.append(torch.zeros(shape, dtype=dt, device=ex.device))
        else:
            vals.append(torch.empty(shape, dtype=dt, device=ex.device))
    env[op.outputs[0]] = vals


OpDef("init", infer=_infer_init, special=_special_init)


def init(shape: Iterable[int], dtype: _dtype, name: Optional[str] = None, init_type: str = "zero",
         meta_shape: Optional[Iterable[int]] = None) -> Tensor:
    """Fresh tensor in the current graph: `"zero"`-filled or `"undef"` (uninitialised)."""
    return emit("init", [], {"shape": tuple(shape), "dt": _dtype.as_dtype(dtype), "init_type": init_type,
                             "meta_shape": tuple(meta_shape) if meta_shape else ()}, [name or "init"])[0]


def _split_seed_ref(seed):
    if seed.device.type == "meta":
        return seed.clone(), seed.clone()
    s = seed.to(torch.int64) & 0xFFFFFFFF
    a = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFF
    b = (s * 2862933555777941757 + 3037000493) & 0xFFFFFFFF
    return a.to(seed.dtype), b.to(seed.dtype)


OpDef("split_random_seed", impl=_split_seed_ref)


def split_random_seed(seed: Tensor, n: int = 2) -> Tuple[Tensor, ...]:
    """Derive `n` new seeds from `seed` (counter-free LCG mixing; deterministic and replica-independent)."""
    outs = []
    cur = seed
    for _ in range(n - 1):
        cur, nxt = emit("split_random_seed", [cur])
        outs.append(nxt)
    return tuple([cur] + outs)


def _seeded_gen(seed: torch.Tensor) -> torch.Generator:
    g = torch.Generator(device=seed.device)
    g.manual_seed(int(seed.reshape(-1).to(torch.int64).sum().item()) & 0x7FFFFFFF)
    return g


def _dropout_ref(x, seed, p):
    if x.device.type == "meta":
        return torch.empty_like(x), torch.empty(x.shape, dtype=torch.bool, device="meta")
    mask = torch.rand(x.shape, generator=_seeded_gen(seed), device=x.device) >= p
    return (x * mask.to(x.dtype) / (1.0 - p)), mask


OpDef("dropout", impl=_dropout_ref,
      vjp=lambda ctx, op, gs: [mul(mul(gs[0], cast(ctx.fwd(op.outputs[1]), gs[0].dtype)),
                                   _const_like(1.0 / (1.0 - op.attrs["p"]), gs[0])), None])


def dropout(t: Tensor, seed_tensor: Tensor, p: float) -> Tensor:
    if p <= 0.0:
        return t
    return emit("dropout", [t, seed_tensor], {"p": float(p)})[0]


def _random_ref(kind):
    def f(seed, shape, dt, a, b):
        if seed.device.type == "meta":
            return torch.empty(shape, dtype=dt.as_torch(), device="meta")
        gen = _seeded_gen(seed)
        if kind == "normal":
            out = torch.randn(shape, generator=gen, device=seed.device) * b + a
        else:
            out = torch.rand(shape, generator=gen, device=seed.device) * (b - a) + a
        return out.to(dt.as_torch())

    return f


OpDef("random_normal", impl=_random_ref("normal"))
OpDef("random_uniform", impl=_random_ref("uniform"))


def random_normal(seed_tensor: Tensor, shape, mean: float = 0.0, std: float = 1.0, dtype=_dt.float32) -> Tensor:
    return emit1("random_normal", [seed_tensor], {"shape": tuple(shape), "dt": _dtype.as_dtype(dtype),
                                                  "a": mean, "b": std})


def random_uniform(seed_tensor: Tensor, shape, low: float = 0.0, high: float = 1.0, dtype=_dt.float32) -> Tensor:
    return emit1("random_uniform", [seed_tensor], {"shape": tuple(shape), "dt": _dtype.as_dtype(dtype),
                                                   "a": low, "b": high})


# ===============================================================================================================
# losses
# ===============================================================================================================


def _nll_ref(probs, labels, ignore_index, reduction, log_prob):
    p = probs.float()
    logp = p if log_prob else torch.log(p)
    return _nll_from_logp(logp, labels, ignore_index, reduction).to(probs.dtype)


def _nll_from_logp(logp, labels, ignore_index, reduction):
    lab = labels.long()
    ii = -100 if ignore_index is None else ignore_index
    flat = logp.reshape(-1, logp.shape[-1])
    return F.nll_loss(flat, lab.reshape(-1), ignore_index=ii, reduction=reduction if reduction != "none" else "none") \
        .reshape(lab.shape if reduction == "none" else ())


def _nll_grad_ref(probs, labels, g, ignore_index, reduction, log_prob):
    with torch.enable_grad():
        pr = probs.detach().float().requires_grad_(True)
        logp = pr if log_prob else torch.log(pr)
        loss = _nll_from_logp(logp, labels, ignore_index, reduction)
        (dp,) = torch.autograd.grad(loss, pr, g.float().reshape(loss.shape))
    return dp.to(probs.dtype)


OpDef("nll_loss", impl=_nll_ref,
      vjp=lambda ctx, op, gs: [emit1("nll_loss_grad", [ctx.fwd(op.inputs[0]), ctx.fwd(op.inputs[1]), gs[0]],
                                     dict(op.attrs)), None])
OpDef("nll_loss_grad", impl=_nll_grad_ref, infer=_infer_like_inputs(1))


def nll_loss(probs: Tensor, labels: Tensor, ignore_index: Optional[int] = None, reduction: str = "mean",
             log_prob: bool = False) -> Tensor:
    return emit1("nll_loss", [probs, labels], {"ignore_index": ignore_index, "reduction": reduction,
                                               "log_prob": log_prob})


def _nll_softmax_grad_ref(probs, labels, loss_grad, ignore_index, reduction):
    """Loss from probabilities and, fused, d(loss)/d(logits) = (p - onehot) * upstream (scaled for `mean`)."""
    p = probs.float()
    lab = labels.long().reshape(-1)
    flat = p.reshape(-1, p.shape[-1])
    ii = -100 if ignore_index is None else ignore_index
    valid = lab != ii
    safe = lab.clamp(0, flat.shape[-1] - 1)
    picked = flat.gather(1, safe.unsqueeze(1)).squeeze(1)
    nll = -torch.log(picked) * valid.float()
    onehot = torch.zeros_like(flat).scatter_(1, safe.unsqueeze(1), 1.0)
    dlogits = (flat - onehot) * valid.float().unsqueeze(1)
    lg = loss_grad.float().reshape(())
    if reduction == "mean":
        denom = valid.float().sum().clamp(min=1.0)
        loss = nll.sum() / denom
        dlogits = dlogits * (lg / denom)
    elif reduction == "sum":
        loss = nll.sum()
        dlogits = dlogits * lg
    else:
        loss = nll.reshape(labels.shape)
        dlogits = dlogits * lg
    return loss.to(probs.dtype), dlogits.reshape(probs.shape).to(probs.dtype)


OpDef("nll_loss_with_softmax_grad", impl=_nll_softmax_grad_ref)


def nll_loss_with_softmax_grad(probs: Tensor, labels: Tensor, loss_grad=1.0, reduction: str = "mean",
                               ignore_index: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    if not isinstance(loss_grad, Tensor):
        loss_grad = constant(loss_grad, _dt.float32)
    loss, dlogits = emit("nll_loss_with_softmax_grad", [probs, labels, loss_grad],
                         {"ignore_index": ignore_index, "reduction": reduction})
    return loss, dlogits


# ===============================================================================================================
# FP8 helpers
# ===============================================================================================================

_FP8_MAX = {"float8_143": 448.0, "float8_152": 57344.0}  # OCP e4m3fn / e5m2 finite maxima


def _pow2cast_to_fp8_ref(x, log2_scale, dt):
    if x.device.type == "meta":
        return torch.empty(x.shape, dtype=dt.as_torch(), device="meta")
    s = torch.exp2(log2_scale.float())
    lim = _FP8_MAX[dt.name]
    return (x.float() * s).clamp(-lim, lim).to(dt.as_torch())


def _pow2cast_from_fp8_ref(x, log2_scale, dt):
    if x.device.type == "meta":
        return torch.empty(x.shape, dtype=dt.as_torch(), device="meta")
    return (x.float() * torch.exp2(log2_scale.float())).to(dt.as_torch())


OpDef("pow2scale_cast_to_fp8", impl=_pow2cast_to_fp8_ref)
OpDef("pow2scale_cast_from_fp8", impl=_pow2cast_from_fp8_ref)


def pow2scale_cast_to_fp8(t: Tensor, log2_scale: Tensor, data_type: _dtype = _dt.float8_143) -> Tensor:
    """`saturate(t * 2**log2_scale)` cast to an 8-bit float."""
    return emit1("pow2scale_cast_to_fp8", [t, log2_scale], {"dt": _dtype.as_dtype(data_type)})


def pow2scale_cast_from_fp8(t: Tensor, log2_scale: Tensor, data_type: _dtype = _dt.float16) -> Tensor:
    return emit1("pow2scale_cast_from_fp8", [t, log2_scale], {"dt": _dtype.as_dtype(data_type)})


def _mm_pow2_ref(a, b, log2_scale, out_dt):
    if a.device.type == "meta":
        return torch.empty((*a.shape[:-1], b.shape[-1]), dtype=out_dt.as_torch(), device="meta")
    y = torch.matmul(a.float(), b.float()) * torch.exp2(log2_scale.float())
    return y.to(out_dt.as_torch())


OpDef("matmul_pow2scaled", impl=_mm_pow2_ref)


def matmul_pow2scaled(lhs: Tensor, rhs: Tensor, log2_scale: Tensor, output_type: _dtype = _dt.float16) -> Tensor:
    """FP8 x FP8 GEMM with fp32 accumulation; the result is multiplied by `2**log2_scale` before the output cast."""
    return emit1("matmul_pow2scaled", [lhs, rhs, log2_scale], {"out_dt": _dtype.as_dtype(output_type)})


# ===============================================================================================================
# debugging
# ===============================================================================================================


def _special_print(ex, op, env):
    vals = env[op.inputs[0]]
    title = op.attrs.get("title") or op.inputs[0].id
    for r, v in enumerate(vals):
        print(f"{title} [replica {ex.global_replica(r)}]: {v}")
    env[op.outputs[0]] = vals


OpDef("print_tensor", special=_special_print, infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, ())],
      vjp=lambda ctx, op, gs: [gs[0]])


def print_tensor(t: Tensor, title: Optional[str] = None, print_self: bool = True, print_gradient: bool = False,
                 summarise_threshold=None, edge_items=None, max_line_width=None, digits=None, float_format=None,
                 separator=None, open_bracket=None, close_bracket=None) -> Tensor:
    return emit1("print_tensor", [t], {"title": title})


# ===============================================================================================================
# sub-graph ops, host IO, remote buffers, device copies: defined in their own modules, re-exported here
# ===============================================================================================================

from .control import (CallSiteInfo, RepeatSiteInfo, call, call_with_info, repeat, repeat_with_info,  # noqa: E402
                      conditional)
from .io import (host_load, host_store, remote_load, remote_load_, remote_store, ipu_copy)  # noqa: E402
from . import var_updates, collectives  # noqa: E402
from .fused import (attention, attention_decode, attention_qkv, rotary_pos_embed, linear_bias_act)  # noqa: E402
from .fused import kv_cache_update_  # noqa: E402


# ---- fused cross-entropy (loss + d loss / d logits in one op) --------------------------------------------------


def _ce_with_grad_ref(logits, labels, loss_grad, ignore_index, reduction):
    probs = torch.softmax(logits.float(), dim=-1).to(logits.dtype) if logits.device.type != "meta" else logits
    if logits.device.type == "meta":
        shape = () if reduction != "none" else labels.shape
        return torch.empty(shape, dtype=logits.dtype, device="meta"), torch.empty_like(logits)
    return _nll_softmax_grad_ref(probs, labels, loss_grad, ignore_index, reduction)


OpDef("ce_with_grad", impl=_ce_with_grad_ref)


def cross_entropy_with_grad(logits: Tensor, labels: Tensor, loss_grad=1.0, reduction: str = "mean",
                            ignore_index: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """Softmax cross-entropy of `logits (.., classes)` against integer `labels`, and its gradient with respect to
    the logits multiplied by `loss_grad`, from one fused pass."""
    if not isinstance(loss_grad, Tensor):
        loss_grad = constant(loss_grad, _dt.float32)
    loss, dlogits = emit("ce_with_grad", [logits, labels, loss_grad],
                         {"ignore_index": ignore_index, "reduction": reduction})
    return loss, dlogits
from .decode import (rotary_kv_append_, attention_decode_packed, argmax_rows, advance_position_, store_row_,  # noqa: E402
                     kv_cache_fill_, timestamp, attention_decode_into_, add_layer_norm_,
                     all_reduce_add_layer_norm_)
from .extra import *  # noqa: E402,F401,F403
# module paths of popxl (`ops.call`, `ops.utils`): loaded here so that a later `from ...ops.call import CallSiteInfo`
# finds the submodule already imported and the name `call` stays bound to the function
from . import utils  # noqa: E402,F401
from .call import call, call_with_info  # noqa: E402,F401,F811
from .conv import conv  # noqa: E402,F401,F811  (`ops.conv` stays the function, `ops.conv.PadType` is reached by path)
from . import negative_log_likelihood  # noqa: E402,F401
