"""Ops of the token-by-token decoding path. The current position lives in a device-side int32 scalar tensor that every
op reads on the device, so a whole decoding step can be captured in a CUDA graph and replayed.

No counterpart in the reference (it ships the int4 `LinearGQ` layer but no generation loop); these ops are what its
GPT-J inference application builds out of `dynamic_update_` / `dynamic_slice` / attention code.
"""
import math
from typing import Optional, Tuple

import torch

from ..core import Tensor
from ..opdef import OPS, OpDef, emit, emit1
from .fused import _rotary_ref


def _pos(p: torch.Tensor) -> int:
    return int(p.reshape(-1)[0].item())


def _rotary_kv_append_ref(qkv, sin_tab, cos_tab, k_cache, v_cache, pos, n_heads, head_dim, rotary_dim):
    if qkv.device.type == "meta":
        return qkv
    p = _pos(pos)
    B = qkv.shape[0]
    hd = n_heads * head_dim
    q = qkv[:, :hd].reshape(B, n_heads, 1, head_dim)
    k = qkv[:, hd:2 * hd].reshape(B, n_heads, 1, head_dim)
    v = qkv[:, 2 * hd:3 * hd].reshape(B, n_heads, 1, head_dim)
    if rotary_dim:
        s, c = sin_tab[p:p + 1].unsqueeze(0), cos_tab[p:p + 1].unsqueeze(0)
        q = _rotary_ref(q, s, c, rotary_dim, False)
        k = _rotary_ref(k, s, c, rotary_dim, False)
        qkv[:, :hd].copy_(q.reshape(B, hd))
        qkv[:, hd:2 * hd].copy_(k.reshape(B, hd))
    k_cache[:, :, p].copy_(k.reshape(B, n_heads, head_dim).to(k_cache.dtype))
    v_cache[:, :, p].copy_(v.reshape(B, n_heads, head_dim).to(v_cache.dtype))
    return qkv


def _attn_decode_packed_ref(qkv, k_cache, v_cache, pos, n_heads, head_dim, scale):
    if qkv.device.type == "meta":
        return torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device="meta")
    L = _pos(pos) + 1
    B = qkv.shape[0]
    q = qkv[:, :n_heads * head_dim].reshape(B, n_heads, 1, head_dim).float()
    s = torch.matmul(q, k_cache[:, :, :L].float().transpose(-1, -2)) * scale
    o = torch.matmul(torch.softmax(s, dim=-1), v_cache[:, :, :L].float())
    return o.reshape(B, n_heads * head_dim).to(qkv.dtype)


def _argmax_rows_ref(logits, valid, index_offset):
    if logits.device.type == "meta":
        return (torch.empty(logits.shape[:-1], dtype=torch.float32, device="meta"),
                torch.empty(logits.shape[:-1], dtype=torch.int32, device="meta"))
    m, i = logits[..., :valid].float().max(dim=-1)
    return m, (i + index_offset).to(torch.int32)


def _advance_ref(pos):
    if pos.device.type != "meta":
        pos.add_(1)
    return pos


def _store_row_ref(buf, pos, vals, base):
    if buf.device.type == "meta":
        return buf
    r = _pos(pos) - base
    if 0 <= r < buf.shape[0]:
        buf[r].copy_(vals)
    return buf


def _kv_fill_ref(rot, k_cache, v_cache, seq_len, n_heads, head_dim):
    if rot.device.type == "meta":
        return k_cache
    B = rot.shape[0] // seq_len
    hd = n_heads * head_dim
    k = rot[:, hd:2 * hd].reshape(B, seq_len, n_heads, head_dim).permute(0, 2, 1, 3)
    v = rot[:, 2 * hd:].reshape(B, seq_len, n_heads, head_dim).permute(0, 2, 1, 3)
    k_cache[:, :, :seq_len].copy_(k)
    v_cache[:, :, :seq_len].copy_(v)
    return k_cache


def _attn_decode_into_ref(buf, k_cache, v_cache, pos, n_heads, head_dim, out_col, scale):
    if buf.device.type == "meta":
        return buf
    o = _attn_decode_packed_ref(buf, k_cache, v_cache, pos, n_heads, head_dim, scale)
    buf[:, out_col:out_col + n_heads * head_dim].copy_(o)
    return buf


def _add_layer_norm_ref(x, *rest, has_delta, has_bias, eps):
    if x.device.type == "meta":
        return torch.empty_like(x)
    rest = list(rest)
    delta = rest.pop(0) if has_delta else None
    bias = rest.pop(0) if has_bias else None
    w, b = rest
    if delta is not None or bias is not None:
        t = x.float()
        if delta is not None:
            t = t + delta.float()
        if bias is not None:
            t = t + bias.float()
        x.copy_(t.to(x.dtype))
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


OpDef("attention_decode_into_", impl=_attn_decode_into_ref, inplace=True)
OpDef("add_layer_norm_", impl=_add_layer_norm_ref)
OpDef("rotary_kv_append_", impl=_rotary_kv_append_ref, inplace=True)
OpDef("attention_decode_packed", impl=_attn_decode_packed_ref)
OpDef("argmax_rows", impl=_argmax_rows_ref)
OpDef("advance_position_", impl=_advance_ref, inplace=True)
OpDef("store_row_", impl=_store_row_ref, inplace=True)
OpDef("kv_cache_fill_", impl=_kv_fill_ref, inplace=True)


def rotary_kv_append_(qkv: Tensor, sin_table: Tensor, cos_table: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor,
                      n_heads: int, head_dim: int, rotary_dim: int) -> Tensor:
    """New-token projections `qkv (batch, 3*heads*head_dim)`: rotate q and k for position `pos` (tables are
    `(max_seq, rotary_dim/2)`) in place and write k, v into the caches `(batch, heads, max_seq, head_dim)` at `pos`."""
    return emit1("rotary_kv_append_", [qkv, sin_table, cos_table, k_cache, v_cache, pos],
                 dict(n_heads=int(n_heads), head_dim=int(head_dim), rotary_dim=int(rotary_dim)))


def attention_decode_packed(qkv: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, n_heads: int, head_dim: int,
                            scale: Optional[float] = None) -> Tensor:
    """Attention of the new query (the q part of `qkv`) against cache positions `[0, pos]`; `(batch, heads*head_dim)`."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    return emit1("attention_decode_packed", [qkv, k_cache, v_cache, pos],
                 dict(n_heads=int(n_heads), head_dim=int(head_dim), scale=scale))


def attention_decode_into_(buf: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, n_heads: int, head_dim: int,
                           out_col: int, scale: Optional[float] = None) -> Tensor:
    """Like `attention_decode_packed` with the query in the first `heads*head_dim` columns of `buf`, but the result is
    written into `buf[:, out_col : out_col + heads*head_dim]` (so that it sits next to other inputs of the following
    linear layer)."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    return emit1("attention_decode_into_", [buf, k_cache, v_cache, pos],
                 dict(n_heads=int(n_heads), head_dim=int(head_dim), out_col=int(out_col), scale=scale))


def add_layer_norm_(x: Tensor, delta: Optional[Tensor], bias: Optional[Tensor], weight: Tensor, ln_bias: Tensor,
                    eps: float = 1e-5) -> Tensor:
    """Residual update fused with the following LayerNorm: `x += delta (+ bias)` in place (skipped when both are None),
    returns `layer_norm(x) * weight + ln_bias`."""
    ins = [x] + ([delta] if delta is not None else []) + ([bias] if bias is not None else []) + [weight, ln_bias]
    return emit1("add_layer_norm_", ins, dict(has_delta=delta is not None, has_bias=bias is not None, eps=float(eps)))


def _special_ar_add_layer_norm(ex, op, env):
    a = op.attrs
    vals = [env[t] for t in op.inputs]
    native = ex.native_collective("ar_add_layer_norm")
    if native is not None:
        res = native(ex, op, *vals)
        if res is not NotImplemented:
            env[op.outputs[0]] = res
            return
    # composition: all-reduce of the partial update, then the residual + LayerNorm op
    vals[1] = ex.comm.all_reduce(vals[1], a["group"], "add")
    od = OPS["add_layer_norm_"]
    fn = od.native.get(ex.device.type) if ex.use_native else None
    kw = dict(has_delta=True, has_bias=a["has_bias"], eps=a["eps"])
    outs = []
    for r in range(ex.num_local):
        args = [v[r] for v in vals]
        res = fn(*args, **kw) if fn is not None else NotImplemented
        if res is NotImplemented:
            res = od.impl(*args, **kw)
        outs.append(res)
    env[op.outputs[0]] = outs


OpDef("all_reduce_add_layer_norm_", special=_special_ar_add_layer_norm, collective=True,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, ())])


def all_reduce_add_layer_norm_(x: Tensor, delta_partial: Tensor, bias: Optional[Tensor], weight: Tensor, ln_bias: Tensor,
                               group, eps: float = 1e-5) -> Tensor:
    """`add_layer_norm_(x, all_reduce(delta_partial, group), bias, ...)` as one op: on one process per GPU the sum over
    the group, the residual update and the LayerNorm run in a single kernel."""
    ins = [x, delta_partial] + ([bias] if bias is not None else []) + [weight, ln_bias]
    return emit1("all_reduce_add_layer_norm_", ins, dict(group=group, has_bias=bias is not None, eps=float(eps)))


def argmax_rows(logits: Tensor, valid: Optional[int] = None, index_offset: int = 0) -> Tuple[Tensor, Tensor]:
    """Per row: maximum over the first `valid` columns (fp32) and its column index plus `index_offset` (int32)."""
    m, i = emit("argmax_rows", [logits], dict(valid=int(valid or logits.shape[-1]), index_offset=int(index_offset)))
    return m, i


def advance_position_(pos: Tensor) -> Tensor:
    return emit1("advance_position_", [pos])


def store_row_(buf: Tensor, pos: Tensor, vals: Tensor, base: int = 0) -> Tensor:
    """`buf[pos - base] = vals` (ignored when the row is out of range)."""
    return emit1("store_row_", [buf, pos, vals], dict(base=int(base)))


def kv_cache_fill_(qkv_rot: Tensor, k_cache: Tensor, v_cache: Tensor, seq_len: int, n_heads: int,
                   head_dim: int) -> Tensor:
    """Copy the (rotated) keys and values of a whole prompt `(batch*seq, 3*heads*head_dim)` into the caches."""
    return emit1("kv_cache_fill_", [qkv_rot, k_cache, v_cache],
                 dict(seq_len=int(seq_len), n_heads=int(n_heads), head_dim=int(head_dim)))


def _special_timestamp(ex, op, env):
    ex.record_timestamp(op.attrs["name"])


OpDef("timestamp", special=_special_timestamp, infer=lambda op: [])


def timestamp(name: str) -> None:
    """Record a device timestamp under `name` at this point of the program (`Session.elapsed_ms(a, b)`)."""
    emit("timestamp", [], {"name": name})
