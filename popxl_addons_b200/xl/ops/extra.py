"""The less-travelled part of the popxl op surface: pooling, resizing, scatter, bit operations, a few reductions,
histogram, shaped dropout, transposed convolution, image normalisation, in-place spellings.

None of these is on a hot path of the add-ons (the reference's layers, transforms and tests do not call them); they are
here so that programs written against popxl find them. Each runs as the PyTorch expression of its definition on
either backend; the gradient ops differentiate that expression with torch.autograd, recomputing the forward from the
op's inputs. Parity: popxl `ops.{scatter, tied_gather, average_pool, max_pool, interpolate, batch_norm_inference,
bitwise_*, logsum, logsumexp, median, histogram, subsample, shaped_dropout, conv_transpose, normalize_image, roi_align,
exp_, relu_, swish_, detach_}`.
"""
from typing import Iterable, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F

from ..core import Tensor
from .. import dtypes as _dt
from ..opdef import OpDef, emit, emit1

__all__ = ["scatter", "tied_gather", "average_pool", "max_pool", "interpolate", "batch_norm_inference", "bitwise_and",
           "bitwise_or", "bitwise_xor", "bitwise_not", "logical_xor", "logsum", "logsumexp", "median", "histogram",
           "subsample", "shaped_dropout", "conv_transpose", "normalize_image", "exp_", "relu_", "swish_", "erf", "nop",
           "detach_", "roi_align"]


def _differentiable(name: str, fn, n_diff: int):
    """Register `name` (computing `fn(*inputs, **attrs)`) with a gradient op for its first `n_diff` inputs."""

    def grad_impl(*args, **attrs):
        *ins, g = args
        if g.device.type == "meta":
            return tuple(torch.empty_like(i) for i in ins[:n_diff])
        with torch.enable_grad():
            leaves = [i.detach().float().requires_grad_(True) for i in ins[:n_diff]]
            y = fn(*leaves, *ins[n_diff:], **attrs)
            grads = torch.autograd.grad(y, leaves, g.to(y.dtype), allow_unused=True)
        return tuple((torch.zeros_like(i) if d is None else d.to(i.dtype)) for d, i in zip(grads, ins))

    def vjp(ctx, op, gs):
        outs = emit(name + "_grad", [ctx.fwd(i) for i in op.inputs] + [gs[0]], dict(op.attrs))
        return list(outs) + [None] * (len(op.inputs) - n_diff)

    OpDef(name, impl=fn, vjp=vjp)
    OpDef(name + "_grad", impl=grad_impl, infer=lambda op: [(t.shape, t.dtype, ()) for t in op.inputs[:n_diff]])


# ---- scatter / tied gather -----------------------------------------------------------------------------------


def _scatter_ref(t, indices, values, dim):
    return t.scatter(dim, indices.long(), values.to(t.dtype))


_differentiable("scatter", lambda t, values, indices, dim: _scatter_ref(t, indices, values, dim), 2)


def scatter(t: Tensor, dim: int, indices: Tensor, values: Tensor, available_memory_proportion=None) -> Tensor:
    """Copy of `t` with `values` written at `indices` along `dim` (`out[indices[i][j]][j] = values[i][j]` for dim 0).
    Gradients flow to `t` (zero at overwritten positions) and to `values`."""
    return emit1("scatter", [t, values, indices], {"dim": dim % t.rank})


def tied_gather(t: Tensor, indices: Tensor, axis: int = 0, available_memory_proportion=None,
                zero_OOR: bool = False) -> Tensor:
    """`gather` for an embedding matrix that is also used, transposed, by the output projection. The reference
    substrate picks a different memory plan for it; the values and gradients are those of `gather`."""
    from . import gather

    return gather(t, indices, axis=axis, zero_OOR=zero_OOR)


# ---- pooling / resize / conv transpose -------------------------------------------------------------------------


def _pads(padding, n):
    """popxl padding: (begin_0, ..., begin_{n-1}, end_0, ..., end_{n-1}) -> F.pad order (last dim first)."""
    padding = tuple(padding) if padding is not None else (0,) * (2 * n)
    out = []
    for d in reversed(range(n)):
        out += [padding[d], padding[n + d]]
    return out


def _avg_pool_ref(x, kernel_size, stride, padding, ceil_mode, count_include_pad):
    n = len(kernel_size)
    fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[n]
    pads = _pads(padding, n)
    sym = all(pads[2 * i] == pads[2 * i + 1] for i in range(n))
    if sym:
        return fn(x, kernel_size, stride, tuple(pads[2 * i] for i in reversed(range(n))), ceil_mode, count_include_pad)
    if not count_include_pad:
        ones = F.pad(torch.ones_like(x), pads)
        return fn(F.pad(x, pads), kernel_size, stride, 0, ceil_mode) / fn(ones, kernel_size, stride, 0, ceil_mode)
    return fn(F.pad(x, pads), kernel_size, stride, 0, ceil_mode)


_differentiable("average_pool", _avg_pool_ref, 1)


def average_pool(t: Tensor, kernel_size: Sequence[int], stride: Optional[Sequence[int]] = None,
                 padding: Optional[Sequence[int]] = None, out_pads=None, out_shape=None, ceil_mode: bool = False,
                 pad_type: str = "not_set", count_include_pad: bool = False) -> Tensor:
    """Average pooling over the trailing `len(kernel_size)` axes of `(N, C, *spatial)`; padding is
    `(begin..., end...)`; padded positions are left out of the mean."""
    k = tuple(int(v) for v in kernel_size)
    return emit1("average_pool", [t], {"kernel_size": k, "stride": tuple(stride) if stride else (1,) * len(k),
                                       "padding": tuple(padding) if padding else (0,) * (2 * len(k)),
                                       "ceil_mode": bool(ceil_mode), "count_include_pad": bool(count_include_pad)})


def _max_pool_ref(x, kernel_size, stride, padding, ceil_mode, dilation):
    n = len(kernel_size)
    fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[n]
    pads = _pads(padding, n)
    if any(pads):
        x = F.pad(x, pads, value=float("-inf"))
    return fn(x, kernel_size, stride, 0, dilation, ceil_mode)


_differentiable("max_pool", _max_pool_ref, 1)


def max_pool(t: Tensor, kernel_size: Sequence[int], stride: Optional[Sequence[int]] = None,
             padding: Optional[Sequence[int]] = None, out_pads=None, out_shape=None, ceil_mode: bool = False,
             pad_type: str = "not_set", storage_order: int = 0, dilation: Optional[Sequence[int]] = None) -> Tensor:
    k = tuple(int(v) for v in kernel_size)
    return emit1("max_pool", [t], {"kernel_size": k, "stride": tuple(stride) if stride else (1,) * len(k),
                                   "padding": tuple(padding) if padding else (0,) * (2 * len(k)),
                                   "ceil_mode": bool(ceil_mode),
                                   "dilation": tuple(dilation) if dilation else (1,) * len(k)})


def _interpolate_ref(x, scale_factor, mode):
    spatial = tuple(float(s) for s in scale_factor[2:])
    size = [int(d * s) for d, s in zip(x.shape[2:], spatial)]
    kw = {} if mode == "nearest" else {"align_corners": False}
    torch_mode = {"nearest": "nearest", "linear": {1: "linear", 2: "bilinear", 3: "trilinear"}.get(len(size)),
                  "cubic": "bicubic"}[mode]
    return F.interpolate(x, size=size, mode=torch_mode, **kw)


_differentiable("interpolate", _interpolate_ref, 1)


def interpolate(t: Tensor, scale_factor: Sequence[float] = (1.0, 1.0, 1.0, 1.0), mode: str = "nearest",
                nearest_mode: str = "round_prefer_floor", coordinate_transformation_mode: str = "half_pixel") -> Tensor:
    """Resize the spatial axes of `(N, C, *spatial)` by `scale_factor` (one factor per axis, batch and channel factors
    must be 1): `nearest`, `linear` or `cubic` with half-pixel centres."""
    sf = tuple(float(s) for s in scale_factor)
    if len(sf) != t.rank or sf[0] != 1.0 or sf[1] != 1.0:
        raise ValueError("scale_factor needs one entry per axis, with 1 for the batch and channel axes")
    if mode not in ("nearest", "linear", "cubic"):
        raise ValueError(f"Unknown interpolation mode {mode}")
    return emit1("interpolate", [t], {"scale_factor": sf, "mode": mode})


def _conv_transpose_ref(x, w, stride, padding, dilation, groups, output_padding):
    n = len(stride)
    pads = tuple(padding) if padding else (0,) * (2 * n)
    if any(pads[d] != pads[n + d] for d in range(n)):
        raise ValueError("conv_transpose takes symmetric padding")
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[n]
    return fn(x, w.to(x.dtype), None, stride, pads[:n], output_padding, groups, dilation)


_differentiable("conv_transpose", _conv_transpose_ref, 2)


def conv_transpose(t: Tensor, weight: Tensor, stride: Sequence[int] = (1, 1), padding: Sequence[int] = (0, 0, 0, 0),
                   dilation: Sequence[int] = (1, 1), groups: int = 1, pad_type: str = "not_set",
                   output_padding: Sequence[int] = (), output_shape: Sequence[int] = (), **planner_options) -> Tensor:
    """Transposed convolution of `(N, C_in, *spatial)` with `weight (C_in, C_out / groups, *kernel)`."""
    n = len(stride)
    return emit1("conv_transpose", [t, weight],
                 {"stride": tuple(stride), "padding": tuple(padding), "dilation": tuple(dilation), "groups": int(groups),
                  "output_padding": tuple(output_padding) if output_padding else (0,) * n})


def _bn_inf_ref(x, scale, bias, mean, var, epsilon):
    shape = [1, -1] + [1] * (x.dim() - 2)
    inv = torch.rsqrt(var.float() + epsilon) * scale.float()
    return ((x.float() - mean.float().reshape(shape)) * inv.reshape(shape) + bias.float().reshape(shape)).to(x.dtype)


_differentiable("batch_norm_inference", _bn_inf_ref, 3)


def batch_norm_inference(t: Tensor, scale: Tensor, bias: Tensor, mean: Tensor, var: Tensor, epsilon: float = 1e-5,
                         momentum: float = 0.9) -> Tensor:
    """Batch normalisation over axis 1 with the given (fixed) statistics."""
    return emit1("batch_norm_inference", [t, scale, bias, mean, var], {"epsilon": float(epsilon)})


def _normalize_image_ref(img, offsets, scales, scale):
    pad = F.pad(img, (0, 4 - img.shape[-1]))
    off = F.pad(offsets.to(img.dtype), (0, 1))
    sc = F.pad(scales.to(img.dtype), (0, 1))
    return (pad * scale - off) * sc


OpDef("normalize_image", impl=_normalize_image_ref)


def normalize_image(image: Tensor, scale: float, offsets: Tensor, scales: Tensor) -> Tensor:
    """Pad a channels-last 3-channel image to 4 channels and compute `(image * scale - offsets) * scales`."""
    if image.shape[-1] != 3:
        raise ValueError("normalize_image takes a channels-last image with 3 channels")
    return emit1("normalize_image", [image, offsets, scales], {"scale": float(scale)})


# ---- bit and logic ops -----------------------------------------------------------------------------------------

for _n, _f in (("bitwise_and", torch.bitwise_and), ("bitwise_or", torch.bitwise_or), ("bitwise_xor", torch.bitwise_xor),
               ("logical_xor", torch.logical_xor)):
    OpDef(_n, impl=_f)
OpDef("bitwise_not", impl=torch.bitwise_not)


def bitwise_and(lhs: Tensor, rhs: Tensor) -> Tensor:
    return emit1("bitwise_and", [lhs, rhs])


def bitwise_or(lhs: Tensor, rhs: Tensor) -> Tensor:
    return emit1("bitwise_or", [lhs, rhs])


def bitwise_xor(lhs: Tensor, rhs: Tensor) -> Tensor:
    return emit1("bitwise_xor", [lhs, rhs])


def logical_xor(lhs: Tensor, rhs: Tensor) -> Tensor:
    return emit1("logical_xor", [lhs, rhs])


def bitwise_not(t: Tensor) -> Tensor:
    return emit1("bitwise_not", [t])


# ---- reductions ------------------------------------------------------------------------------------------------


def _axes(t: Tensor, axis) -> Tuple[int, ...]:
    if axis is None:
        return tuple(range(t.rank))
    if isinstance(axis, int):
        axis = (axis,)
    return tuple(sorted(a % t.rank for a in axis))


_differentiable("logsum", lambda a, axes, keepdims: torch.log(torch.sum(a, dim=axes, keepdim=keepdims)), 1)
_differentiable("logsumexp", lambda a, axes, keepdims: torch.logsumexp(a, dim=axes, keepdim=keepdims), 1)


def logsum(t: Tensor, axis: Optional[Union[int, Iterable[int]]] = None, keepdims: bool = False) -> Tensor:
    """`log(sum(t))` over `axis` (all axes by default)."""
    return emit1("logsum", [t], {"axes": _axes(t, axis), "keepdims": bool(keepdims)})


def logsumexp(t: Tensor, axis: Optional[Union[int, Iterable[int]]] = None, keepdims: bool = False) -> Tensor:
    return emit1("logsumexp", [t], {"axes": _axes(t, axis), "keepdims": bool(keepdims)})


def _median_ref(a, axes, keepdims):
    keep = [d for d in range(a.dim()) if d not in axes]
    flat = a.permute(*keep, *axes).reshape(*[a.shape[d] for d in keep], -1)
    out = flat.median(dim=-1).values
    if keepdims:
        out = out.reshape([1 if d in axes else a.shape[d] for d in range(a.dim())])
    return out


_differentiable("median", _median_ref, 1)


def median(t: Tensor, axis: Optional[Union[int, Iterable[int]]] = None, keepdims: bool = False) -> Tensor:
    """Median over `axis` (the lower of the two middle values for an even count)."""
    return emit1("median", [t], {"axes": _axes(t, axis), "keepdims": bool(keepdims)})


def _histogram_ref(a, levels, absolute_of_input):
    if a.device.type == "meta":
        return torch.empty(len(levels) + 1, dtype=torch.uint32, device="meta")
    v = a.float().reshape(-1)
    if absolute_of_input:
        v = v.abs()
    edges = torch.tensor(levels, dtype=torch.float32, device=a.device)
    bins = torch.bucketize(v, edges, right=True)  # bin i holds levels[i-1] <= x < levels[i]
    return torch.bincount(bins, minlength=len(levels) + 1).to(torch.uint32)


OpDef("histogram", impl=_histogram_ref)


def histogram(t: Tensor, levels: List[float], absolute_of_input: bool = False) -> Tensor:
    """Counts of the elements of `t` in the `len(levels) + 1` bins `(-inf, l0), [l0, l1), ..., [l_last, inf)`
    (of `|t|` if `absolute_of_input`), as uint32."""
    lv = tuple(float(v) for v in levels)
    if list(lv) != sorted(lv):
        raise ValueError("histogram levels must ascend")
    return emit1("histogram", [t], {"levels": lv, "absolute_of_input": bool(absolute_of_input)})


def _subsample_ref(a, strides):
    return a[tuple(slice(None, None, s) for s in strides)]


_differentiable("subsample", _subsample_ref, 1)


def subsample(t: Tensor, slices: Union[int, Sequence[int]]) -> Tensor:
    """Every `slices[d]`-th element along axis `d` (one stride for all axes if an int)."""
    st = (int(slices),) * t.rank if isinstance(slices, int) else tuple(int(s) for s in slices)
    if len(st) != t.rank or any(s < 1 for s in st):
        raise ValueError("subsample needs one positive stride per axis")
    return emit1("subsample", [t], {"strides": st})


# ---- shaped dropout --------------------------------------------------------------------------------------------


def _shaped_dropout_ref(x, seed, shape, ratio):
    if x.device.type == "meta":
        return torch.empty_like(x), torch.empty(shape, dtype=torch.bool, device="meta")
    from . import _seeded_gen

    mask = torch.rand(tuple(shape), generator=_seeded_gen(seed), device=x.device) >= ratio
    return x * mask.to(x.dtype) / (1.0 - ratio), mask


def _shaped_dropout_vjp(ctx, op, gs):
    from . import cast, mul, _const_like

    return [mul(mul(gs[0], cast(ctx.fwd(op.outputs[1]), gs[0].dtype)),
                _const_like(1.0 / (1.0 - op.attrs["ratio"]), gs[0])), None]


OpDef("shaped_dropout", impl=_shaped_dropout_ref, vjp=_shaped_dropout_vjp)


def shaped_dropout(t: Tensor, seed_tensor: Tensor, shape: Iterable[int], ratio: float) -> Tensor:
    """Dropout whose mask has `shape` (broadcastable to `t`): whole rows, channels or feature maps drop together."""
    shape = tuple(int(s) for s in shape)
    try:
        ok = torch.broadcast_shapes(shape, tuple(t.shape)) == tuple(t.shape)
    except RuntimeError:
        ok = False
    if not ok:
        raise ValueError(f"Mask shape {shape} does not broadcast to {tuple(t.shape)}")
    if ratio <= 0.0:
        return t
    return emit("shaped_dropout", [t, seed_tensor], {"shape": shape, "ratio": float(ratio)})[0]


# ---- misc ------------------------------------------------------------------------------------------------------

_differentiable("erf", lambda a: torch.erf(a), 1)


def erf(t: Tensor) -> Tensor:
    return emit1("erf", [t])


def nop(t: Tensor) -> Tensor:
    from . import identity

    return identity(t)


def exp_(t: Tensor) -> Tensor:
    """In-place spellings compute out of place here: buffers are recycled by the allocator, not by the program."""
    from . import exp

    return exp(t)


def relu_(t: Tensor) -> Tensor:
    from . import relu

    return relu(t)


def swish_(t: Tensor) -> Tensor:
    from . import swish

    return swish(t)


def detach_(t: Tensor) -> Tensor:
    from . import detach

    return detach(t)


def _roi_align_ref(x, rois, batch_index, output_size, spatial_scale, sampling_ratio):
    if x.device.type == "meta":
        return torch.empty((rois.shape[0], x.shape[1], *output_size), dtype=x.dtype, device="meta")
    from torchvision.ops import roi_align as _tv_roi_align

    boxes = torch.cat([batch_index.to(x.dtype).reshape(-1, 1), rois.to(x.dtype)], dim=1)
    return _tv_roi_align(x, boxes, tuple(output_size), float(spatial_scale), int(sampling_ratio), aligned=False)


_differentiable("roi_align", _roi_align_ref, 1)


def roi_align(t: Tensor, rois: Tensor, batch_index: Tensor, output_size: Sequence[int], spatial_scale: float,
              sampling_ratio: int) -> Tensor:
    """Region-of-interest align (Mask R-CNN): `t (N, C, H, W)`, `rois (K, 4)` as `(x1, y1, x2, y2)` in input
    coordinates times `1 / spatial_scale`, `batch_index (K,)`; bilinear samples on a `sampling_ratio` grid per output
    bin, averaged. Result `(K, C, *output_size)`."""
    if t.rank != 4 or rois.rank != 2 or rois.shape[1] != 4 or batch_index.shape != (rois.shape[0],):
        raise ValueError("roi_align takes t (N, C, H, W), rois (K, 4) and batch_index (K,)")
    return emit1("roi_align", [t, rois, batch_index],
                 {"output_size": tuple(int(v) for v in output_size), "spatial_scale": float(spatial_scale),
                  "sampling_ratio": int(sampling_ratio)})
