"""Optimizer-state update ops (`xl.ops.var_updates.*`), all in place on their first operand.

Scalars (decay factors, learning rate, ...) may be Python floats baked into the op or scalar tensors read at run time.
Parity: popxl `ops.var_updates.{accumulate_, accumulate_mean_, accumulate_moving_average_,
accumulate_moving_average_square_, accumulator_zero_, accumulator_scale_, adam_updater, copy_var_update_}` used by
popxl_addons/optimizers/adam.py:85-111 and transforms/autodiff.py:189. `adam_fused_` / `sgd_fused_` are the
one-kernel forms the optimizers of this package emit.
"""
from typing import Optional, Union

import torch

from ..core import Tensor
from .. import dtypes as _dt
from ..opdef import OpDef, emit, emit1

Scalar = Union[float, Tensor]


def _pack(inputs, **scalars):
    """Tensor-valued scalars become extra op inputs (in keyword order); floats go into attrs."""
    attrs, order = {}, []
    for k, v in scalars.items():
        if isinstance(v, Tensor):
            inputs.append(v)
            order.append(k)
            attrs[k] = None
        else:
            attrs[k] = v
    attrs["_tensor_scalars"] = tuple(order)
    return inputs, attrs


def _unpack(extra, attrs):
    vals = dict(attrs)
    order = vals.pop("_tensor_scalars")
    for k, t in zip(order, extra):
        vals[k] = t.float().reshape(()) if t.device.type != "meta" else 1.0
    return vals


def _f(x):
    return x.float() if isinstance(x, torch.Tensor) else x


def _accumulate_ref(t, X, *extra, **attrs):
    if t.device.type == "meta":
        return t
    s = _unpack(extra, attrs)
    f = s["f"]
    return t.add_((X.float() * (1.0 if f is None else f)).to(t.dtype))


def _accumulate_mean_ref(t, X, *extra, **attrs):
    if t.device.type == "meta":
        return t
    step = _unpack(extra, attrs)["step"]
    res = t.float() * (step / (step + 1.0)) + X.float() * (1.0 / (step + 1.0))
    return t.copy_(res.to(t.dtype))


def _acc_ma_ref(t, X, *extra, **attrs):
    if t.device.type == "meta":
        return t
    f = _unpack(extra, attrs)["f"]
    return t.copy_((t.float() * f + X.float() * (1.0 - f)).to(t.dtype))


def _acc_ma_sq_ref(t, X, *extra, **attrs):
    if t.device.type == "meta":
        return t
    f = _unpack(extra, attrs)["f"]
    xf = X.float()
    return t.copy_((t.float() * f + xf * xf * (1.0 - f)).to(t.dtype))


def _acc_zero_ref(t):
    if t.device.type == "meta":
        return t
    return t.zero_()


def _acc_scale_ref(t, *extra, **attrs):
    if t.device.type == "meta":
        return t
    f = _unpack(extra, attrs)["f"]
    return t.copy_((t.float() * f).to(t.dtype))


OpDef("accumulate_", impl=_accumulate_ref, inplace=True, keeps_meta=True)
OpDef("accumulate_mean_", impl=_accumulate_mean_ref, inplace=True, keeps_meta=True)
OpDef("accumulate_moving_average_", impl=_acc_ma_ref, inplace=True, keeps_meta=True)
OpDef("accumulate_moving_average_square_", impl=_acc_ma_sq_ref, inplace=True, keeps_meta=True)
OpDef("accumulator_zero_", impl=_acc_zero_ref, inplace=True, keeps_meta=True)
OpDef("accumulator_scale_", impl=_acc_scale_ref, inplace=True, keeps_meta=True)


def accumulate_(t: Tensor, X: Tensor, f: Optional[Scalar] = None) -> Tensor:
    """`t += f * X`."""
    ins, attrs = _pack([t, X], f=f)
    return emit1("accumulate_", ins, attrs)


def accumulate_mean_(t: Tensor, X: Tensor, step: Scalar) -> Tensor:
    """Running mean: `t = t * step/(step+1) + X/(step+1)`."""
    ins, attrs = _pack([t, X], step=step)
    return emit1("accumulate_mean_", ins, attrs)


def accumulate_moving_average_(t: Tensor, X: Tensor, f: Scalar) -> Tensor:
    """`t = f*t + (1-f)*X`."""
    ins, attrs = _pack([t, X], f=f)
    return emit1("accumulate_moving_average_", ins, attrs)


def accumulate_moving_average_square_(t: Tensor, X: Tensor, f: Scalar) -> Tensor:
    """`t = f*t + (1-f)*X^2`."""
    ins, attrs = _pack([t, X], f=f)
    return emit1("accumulate_moving_average_square_", ins, attrs)


def accumulator_zero_(t: Tensor) -> Tensor:
    return emit1("accumulator_zero_", [t])


def accumulator_scale_(t: Tensor, f: Scalar) -> Tensor:
    ins, attrs = _pack([t], f=f)
    return emit1("accumulator_scale_", ins, attrs)


def _acc_square_ref(t, X, *extra, **attrs):
    if t.device.type == "meta":
        return t
    f = _unpack(extra, attrs)["f"]
    xf = X.float()
    return t.add_((xf * xf * (1.0 if f is None else f)).to(t.dtype))


def _sparse_accumulate_ref(t, X, indices, *extra, axis, **attrs):
    if t.device.type == "meta":
        return t
    f = _unpack(extra, attrs)["f"]
    upd = (X.float() * (1.0 if f is None else f)).to(t.dtype)
    return t.index_add_(axis, indices.long().reshape(-1), upd.reshape(*t.shape[:axis], -1, *t.shape[axis + 1:]))


OpDef("accumulate_square_", impl=_acc_square_ref, inplace=True, keeps_meta=True)
OpDef("sparse_accumulate_", impl=_sparse_accumulate_ref, inplace=True, keeps_meta=True)


def accumulate_square_(t: Tensor, X: Tensor, f: Optional[Scalar] = None) -> Tensor:
    """`t += f * X^2`."""
    ins, attrs = _pack([t, X], f=f)
    return emit1("accumulate_square_", ins, attrs)


def sparse_accumulate_(t: Tensor, X: Tensor, indices: Tensor, axis: int = 0, f: Optional[Scalar] = None,
                       W: Optional[Tensor] = None) -> Tensor:
    """`t[indices] += f * X` along `axis`: the accumulator update for the gradient of a gather, touching only the
    gathered rows (`W`, the tied weight the reference substrate uses to pick a layout, is accepted and ignored)."""
    ins, attrs = _pack([t, X, indices], f=f)
    attrs["axis"] = axis % t.rank
    return emit1("sparse_accumulate_", ins, attrs)


def copy_var_update_(t: Tensor, X: Tensor) -> Tensor:
    return emit1("copy_var_update_", [t, X])


# ---- Adam ----------------------------------------------------------------------------------------------------


def _adam_updater_ref(m, v, *rest, has_weight, has_step, **attrs):
    rest = list(rest)
    w = rest.pop(0) if has_weight else None
    step = rest.pop(0) if has_step else None
    if m.device.type == "meta":
        return torch.empty(m.shape, dtype=torch.float32, device="meta")
    s = _unpack(rest, attrs)
    mf, vf = m.float(), v.float()
    if step is not None:
        step.add_(1)
        t = step.float()
        mf = mf / (1.0 - s["beta1"] ** t)
        vf = vf / (1.0 - s["beta2"] ** t)
    upd = mf / (torch.sqrt(vf) + s["epsilon"])
    wd = s["weight_decay"]
    if w is not None and wd is not None and not (isinstance(wd, float) and wd == 0.0):
        upd = upd + w.float() * wd
    return upd


OpDef("adam_updater", impl=_adam_updater_ref, keeps_meta=True)


def adam_updater(acc_first_order: Tensor, acc_second_order: Tensor, weight: Optional[Tensor] = None,
                 time_step: Optional[Tensor] = None, weight_decay: Optional[Scalar] = None,
                 beta1: Optional[Scalar] = None, beta2: Optional[Scalar] = None,
                 epsilon: Scalar = 1e-07) -> Tensor:
    """`m_hat / (sqrt(v_hat) + eps) + wd * w`. With `time_step` the step counter is incremented in place and
    bias correction `m_hat = m / (1 - beta1^t)`, `v_hat = v / (1 - beta2^t)` is applied."""
    if time_step is not None and (beta1 is None or beta2 is None):
        raise ValueError("Bias correction requires both beta1 and beta2")
    if weight_decay is not None and weight is None:
        raise ValueError("Weight decay requires the weight tensor")
    ins = [acc_first_order, acc_second_order]
    if weight is not None:
        ins.append(weight)
    if time_step is not None:
        ins.append(time_step)
    ins, attrs = _pack(ins, weight_decay=weight_decay, beta1=beta1, beta2=beta2, epsilon=epsilon)
    attrs.update(has_weight=weight is not None, has_step=time_step is not None)
    return emit1("adam_updater", ins, attrs)


def _lamb_updater_ref(m, v, *rest, has_weight, has_step, **attrs):
    # the LAMB direction is Adam's, without the learning rate: the trust ratio is applied by the caller
    return _adam_updater_ref(m, v, *rest, has_weight=has_weight, has_step=has_step, **attrs)


def _adamax_updater_ref(m, v, *rest, has_weight, has_step, **attrs):
    rest = list(rest)
    w = rest.pop(0) if has_weight else None
    step = rest.pop(0) if has_step else None
    if m.device.type == "meta":
        return torch.empty(m.shape, dtype=torch.float32, device="meta")
    s = _unpack(rest, attrs)
    mf = m.float()
    if step is not None:
        step.add_(1)
        mf = mf / (1.0 - s["beta1"] ** step.float())
    upd = mf / (v.float() + s["epsilon"])
    wd = s["weight_decay"]
    if w is not None and wd is not None and not (isinstance(wd, float) and wd == 0.0):
        upd = upd + w.float() * wd
    return upd


OpDef("lamb_updater", impl=_lamb_updater_ref, keeps_meta=True)
OpDef("adamax_updater", impl=_adamax_updater_ref, keeps_meta=True)


def lamb_updater(acc_first_order: Tensor, acc_second_order: Tensor, weight: Optional[Tensor] = None,
                 time_step: Optional[Tensor] = None, weight_decay: Optional[Scalar] = None,
                 beta1: Optional[Scalar] = None, beta2: Optional[Scalar] = None, epsilon: Scalar = 1e-07) -> Tensor:
    """The LAMB update direction `m_hat / (sqrt(v_hat) + eps) + wd * w` (to be scaled by `lr * |w| / |direction|`)."""
    if time_step is not None and (beta1 is None or beta2 is None):
        raise ValueError("Bias correction requires both beta1 and beta2")
    if weight_decay is not None and weight is None:
        raise ValueError("Weight decay requires the weight tensor")
    ins = [acc_first_order, acc_second_order] + ([weight] if weight is not None else []) + \
        ([time_step] if time_step is not None else [])
    ins, attrs = _pack(ins, weight_decay=weight_decay, beta1=beta1, beta2=beta2, epsilon=epsilon)
    attrs.update(has_weight=weight is not None, has_step=time_step is not None)
    return emit1("lamb_updater", ins, attrs)


def adamax_updater(acc_first_order: Tensor, acc_second_order: Tensor, weight: Optional[Tensor] = None,
                   time_step: Optional[Tensor] = None, weight_decay: Optional[Scalar] = None,
                   beta1: Optional[Scalar] = None, epsilon: Scalar = 1e-07) -> Tensor:
    """Adamax direction `m_hat / (u + eps) + wd * w`, with `u` the running infinity norm held in
    `acc_second_order`; with `time_step` the counter is incremented and `m` bias-corrected."""
    if time_step is not None and beta1 is None:
        raise ValueError("Bias correction requires beta1")
    if weight_decay is not None and weight is None:
        raise ValueError("Weight decay requires the weight tensor")
    ins = [acc_first_order, acc_second_order] + ([weight] if weight is not None else []) + \
        ([time_step] if time_step is not None else [])
    ins, attrs = _pack(ins, weight_decay=weight_decay, beta1=beta1, epsilon=epsilon)
    attrs.update(has_weight=weight is not None, has_step=time_step is not None)
    return emit1("adamax_updater", ins, attrs)


def _adam_fused_ref(w, g, m, v, *rest, has_step, has_master, bias_correction, **attrs):
    """Whole AdamW step on one tensor: state update, bias correction, decoupled weight decay, weight update."""
    rest = list(rest)
    step = rest.pop(0) if has_step else None
    master = rest.pop(0) if has_master else None
    if w.device.type == "meta":
        return w
    s = _unpack(rest, attrs)
    gf = g.float() * s["grad_scale"]
    mf = m.float() * s["beta1"] + gf * (1.0 - s["beta1"])
    vf = v.float() * s["beta2"] + gf * gf * (1.0 - s["beta2"])
    m.copy_(mf.to(m.dtype))
    v.copy_(vf.to(v.dtype))
    mh, vh = m.float(), vf
    if step is not None:
        step.add_(1)
        if bias_correction:
            t = step.float()
            mh = mh / (1.0 - s["beta1"] ** t)
            vh = vh / (1.0 - s["beta2"] ** t)
    src = master if master is not None else w
    wf = src.float()
    upd = mh / (torch.sqrt(vh) + s["epsilon"]) + wf * s["weight_decay"]
    wf = wf - s["lr"] * upd
    if master is not None:
        master.copy_(wf)
    w.copy_(wf.to(w.dtype))
    return w


OpDef("adam_fused_", impl=_adam_fused_ref, inplace=True, keeps_meta=True)


def adam_fused_(var: Tensor, grad: Tensor, first_order: Tensor, second_order: Tensor,
                step: Optional[Tensor] = None, master: Optional[Tensor] = None, *, lr: Scalar,
                beta1: Scalar = 0.9, beta2: Scalar = 0.999, epsilon: Scalar = 1e-5, weight_decay: Scalar = 0.0,
                grad_scale: Scalar = 1.0, bias_correction: bool = True) -> Tensor:
    """One-kernel AdamW step (same arithmetic as accumulate_moving_average_(_square_) + adam_updater + scaled_add_).
    `master` is an optional fp32 copy of `var` that carries the update when `var` is bf16/fp16."""
    ins = [var, grad, first_order, second_order]
    if step is not None:
        ins.append(step)
    if master is not None:
        ins.append(master)
    ins, attrs = _pack(ins, lr=lr, beta1=beta1, beta2=beta2, epsilon=epsilon, weight_decay=weight_decay,
                       grad_scale=grad_scale)
    attrs.update(has_step=step is not None, has_master=master is not None, bias_correction=bias_correction)
    return emit1("adam_fused_", ins, attrs)


def _sgd_fused_ref(w, g, *rest, has_momentum, **attrs):
    rest = list(rest)
    buf = rest.pop(0) if has_momentum else None
    if w.device.type == "meta":
        return w
    s = _unpack(rest, attrs)
    gf = g.float() * s["grad_scale"] + w.float() * s["weight_decay"]
    if buf is not None:
        bf = buf.float() * s["momentum"] + gf
        buf.copy_(bf.to(buf.dtype))
        gf = bf
    return w.copy_((w.float() - s["lr"] * gf).to(w.dtype))


OpDef("sgd_fused_", impl=_sgd_fused_ref, inplace=True, keeps_meta=True)


def sgd_fused_(var: Tensor, grad: Tensor, momentum_buffer: Optional[Tensor] = None, *, lr: Scalar,
               momentum: Scalar = 0.0, weight_decay: Scalar = 0.0, grad_scale: Scalar = 1.0) -> Tensor:
    """`g' = grad_scale*g + wd*w ; buf = momentum*buf + g' ; w -= lr * buf` (buf omitted without momentum)."""
    ins = [var, grad]
    if momentum_buffer is not None:
        ins.append(momentum_buffer)
    ins, attrs = _pack(ins, lr=lr, momentum=momentum, weight_decay=weight_decay, grad_scale=grad_scale)
    attrs.update(has_momentum=momentum_buffer is not None)
    return emit1("sgd_fused_", ins, attrs)


# ---- weight-gradient GEMM fused with the running-mean accumulation ---------------------------------------------


def _mm_acc_mean_ref(acc, a, b, step):
    if acc.device.type == "meta":
        return acc
    t = step.float().reshape(())
    prod = torch.matmul(a.float(), b.float())
    return acc.copy_((acc.float() * (t / (t + 1.0)) + prod * (1.0 / (t + 1.0))).to(acc.dtype))


OpDef("matmul_accumulate_mean_", impl=_mm_acc_mean_ref, inplace=True, keeps_meta=True,
      flops=lambda op: 2 * op.inputs[1].shape[-1] * op.inputs[0].nelms)


def matmul_accumulate_mean_(acc: Tensor, lhs: Tensor, rhs: Tensor, step: Tensor) -> Tensor:
    """`acc = acc * step/(step+1) + (lhs @ rhs)/(step+1)`: the product never exists in memory, the GEMM epilogue
    folds each output tile into the accumulator (weight gradients under gradient accumulation)."""
    return emit1("matmul_accumulate_mean_", [acc, lhs, rhs, step])
