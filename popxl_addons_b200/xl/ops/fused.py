"""Fused ops that have no single counterpart in the reference's op list but are needed by the transformer
configurations: causal softmax attention (forward saves the log-sum-exp, one fused backward), attention against a
KV cache for decoding, rotary position embedding, and Linear with bias/activation epilogue.

Rotary parity: popxl_addons/ops/rotary_pos_embed/rotary_pos_embedx.cpp:49-70,104-127 (interleaved pairs on the first
`rotary_dim` features; gradient = inverse rotation).
"""
import math
from typing import Optional

import torch

from ..core import Tensor
from ..opdef import OpDef, emit, emit1

# ---- attention -----------------------------------------------------------------------------------------------


def _attn_fwd_ref(q, k, v, causal, scale):
    if q.device.type == "meta":
        return torch.empty_like(q), torch.empty(q.shape[:-1], dtype=torch.float32, device="meta")
    qf, kf, vf = q.float(), k.float(), v.float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(diagonal=sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    return torch.matmul(p, vf).to(q.dtype), lse


def _attn_bwd_ref(q, k, v, o, lse, do, causal, scale):
    if q.device.type == "meta":
        return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    qf, kf, vf, of, dof = q.float(), k.float(), v.float(), o.float(), do.float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(diagonal=sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(dim=-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _vjp_attn(ctx, op, gs):
    q, k, v = op.inputs
    o, lse = op.outputs
    return emit("attention_grad", [ctx.fwd(q), ctx.fwd(k), ctx.fwd(v), ctx.fwd(o), ctx.fwd(lse), gs[0]],
                dict(op.attrs))


def _attn_flops(op):
    b, h, sq, d = op.inputs[0].shape
    sk = op.inputs[1].shape[-2]
    f = 4 * b * h * sq * sk * d
    return f // 2 if op.attrs.get("causal") else f


OpDef("attention", impl=_attn_fwd_ref, vjp=_vjp_attn, flops=_attn_flops)
OpDef("attention_grad", impl=_attn_bwd_ref, flops=lambda op: int(2.5 * _attn_flops(op)))


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, scale: Optional[float] = None) -> Tensor:
    """`softmax(q k^T * scale [+ causal mask]) v` for `(batch, heads, seq, head_dim)` operands."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return emit("attention", [q, k, v], {"causal": bool(causal), "scale": scale})[0]


def _attn_decode_ref(q, k_cache, v_cache, length, scale):
    """q: (B,H,T,D) new tokens; caches: (B,H,Smax,D) already containing the new tokens; `length` = tokens valid
    in the cache *after* the update. Token t of q attends to positions <= length - T + t."""
    if q.device.type == "meta":
        return torch.empty_like(q)
    L = int(length.reshape(-1)[0].item())
    T = q.shape[-2]
    kf, vf = k_cache[..., :L, :].float(), v_cache[..., :L, :].float()
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if T > 1:
        mask = torch.ones(T, L, dtype=torch.bool, device=s.device).tril(diagonal=L - T)
        s = s.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf).to(q.dtype)


OpDef("attention_decode", impl=_attn_decode_ref)


def attention_decode(q: Tensor, k_cache: Tensor, v_cache: Tensor, length: Tensor,
                     scale: Optional[float] = None) -> Tensor:
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return emit1("attention_decode", [q, k_cache, v_cache, length], {"scale": scale})


def _kv_update_ref(cache, new, position):
    if cache.device.type == "meta":
        return cache
    p = int(position.reshape(-1)[0].item())
    cache[..., p:p + new.shape[-2], :].copy_(new)
    return cache


OpDef("kv_cache_update_", impl=_kv_update_ref, inplace=True)


def kv_cache_update_(cache: Tensor, new: Tensor, position: Tensor) -> Tensor:
    """Write `new` `(B,H,T,D)` into `cache` `(B,H,Smax,D)` at sequence offset `position` (in place)."""
    return emit1("kv_cache_update_", [cache, new, position])


# ---- rotary --------------------------------------------------------------------------------------------------


def _rotary_ref(x, sin, cos, rotary_dim, inverse):
    if x.device.type == "meta":
        return torch.empty_like(x)
    xf = x.float()
    rot, rest = xf[..., :rotary_dim], xf[..., rotary_dim:]
    re, im = rot[..., 0::2], rot[..., 1::2]
    s, c = sin.float().unsqueeze(1), cos.float().unsqueeze(1)  # (1|B, 1, S, rot/2)
    if inverse:
        s = -s
    yre = re * c - im * s
    yim = im * c + re * s
    y = torch.stack((yre, yim), dim=-1).flatten(-2)
    return torch.cat((y, rest), dim=-1).to(x.dtype)


def _vjp_rotary(ctx, op, gs):
    x, sin, cos = op.inputs
    a = dict(op.attrs)
    a["inverse"] = not a["inverse"]
    return [emit1("rotary_pos_embed", [gs[0], ctx.fwd(sin), ctx.fwd(cos)], a), None, None]


OpDef("rotary_pos_embed", impl=_rotary_ref, vjp=_vjp_rotary)


def rotary_pos_embed(t: Tensor, sin: Tensor, cos: Tensor, rotary_dim: int) -> Tensor:
    if t.rank != 4:
        raise ValueError(f"rotary_pos_embed expects a rank-4 (batch, heads, seq, head_dim) tensor, got {t.shape}")
    if rotary_dim % 2 or rotary_dim > t.shape[-1]:
        raise ValueError(f"rotary_dim={rotary_dim} must be even and at most the head dimension {t.shape[-1]}")
    if sin.shape != cos.shape or sin.shape[-1] != rotary_dim // 2 or sin.shape[-2] != t.shape[-2]:
        raise ValueError(f"sin/cos must have shape (1|batch, seq, rotary_dim/2); got {sin.shape}, {cos.shape}")
    return emit1("rotary_pos_embed", [t, sin, cos], {"rotary_dim": int(rotary_dim), "inverse": False})


# ---- linear with epilogue ------------------------------------------------------------------------------------


def _lin_ref(x, w, *b, act):
    if x.device.type == "meta":
        return torch.empty((*x.shape[:-1], w.shape[-1]), dtype=x.dtype, device="meta")
    y = torch.matmul(x, w.to(x.dtype))
    if b:
        y = y + b[0].to(y.dtype)
    if act == "gelu":
        y = torch.nn.functional.gelu(y.float()).to(y.dtype)
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(y.float(), approximate="tanh").to(y.dtype)
    elif act == "relu":
        y = torch.relu(y)
    return y


def _vjp_lin(ctx, op, gs):
    from . import matmul, transpose, reshape, sum as _sum, emit1 as _e  # noqa: F401

    if op.attrs["act"] != "none":
        raise NotImplementedError("linear_bias_act with an activation is inference-only; use matmul + gelu to train")
    x, w = op.inputs[0], op.inputs[1]
    g = gs[0]
    fx, fw = ctx.fwd(x), ctx.fwd(w)
    gx = matmul(g, transpose(fw))
    g2 = reshape(g, (-1, g.shape[-1]))
    gw = matmul(transpose(reshape(fx, (-1, x.shape[-1]))), g2)
    out = [gx, gw]
    if len(op.inputs) == 3:
        out.append(_sum(g2, axis=0))
    return out


OpDef("linear_bias_act", impl=_lin_ref, vjp=_vjp_lin,
      flops=lambda op: 2 * op.inputs[0].shape[-1] * op.outputs[0].nelms)


def linear_bias_act(x: Tensor, w: Tensor, b: Optional[Tensor] = None, act: str = "none") -> Tensor:
    """`act(x @ w + b)` as one GEMM with a fused epilogue."""
    ins = [x, w] + ([b] if b is not None else [])
    return emit1("linear_bias_act", ins, {"act": act})


# ---- attention on a packed qkv matrix (the transformer hot path) ----------------------------------------------


def _split_heads(qkv, seq_len, n_heads, head_dim):
    T = qkv.shape[0]
    B = T // seq_len
    hd = n_heads * head_dim
    parts = [qkv[:, i * hd:(i + 1) * hd].reshape(B, seq_len, n_heads, head_dim).permute(0, 2, 1, 3) for i in range(3)]
    return parts, B


def _attn_qkv_fwd_ref(qkv, sin, cos, seq_len, n_heads, head_dim, rotary_dim, causal, scale, inplace):
    if qkv.device.type == "meta":
        T = qkv.shape[0]
        return (torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device="meta"), torch.empty_like(qkv),
                torch.empty((T // seq_len, n_heads, seq_len), dtype=torch.float32, device="meta"))
    (q, k, v), B = _split_heads(qkv, seq_len, n_heads, head_dim)
    if rotary_dim:
        q = _rotary_ref(q, sin, cos, rotary_dim, False)
        k = _rotary_ref(k, sin, cos, rotary_dim, False)
    o, lse = _attn_fwd_ref(q, k, v, causal, scale)
    T = qkv.shape[0]
    rot = torch.cat([t.permute(0, 2, 1, 3).reshape(T, n_heads * head_dim) for t in (q, k, v)], dim=-1).to(qkv.dtype)
    return o.permute(0, 2, 1, 3).reshape(T, n_heads * head_dim), rot, lse


def _attn_qkv_bwd_ref(qkv_rot, lse, dout, sin, cos, *fwd_out, seq_len, n_heads, head_dim, rotary_dim, causal, scale):
    """`fwd_out` (optional): the forward pass's output, which device kernels use for the row sums `dO . O`; this
    reference recomputes it."""
    if qkv_rot.device.type == "meta":
        return torch.empty_like(qkv_rot)
    (q, k, v), B = _split_heads(qkv_rot, seq_len, n_heads, head_dim)
    T = qkv_rot.shape[0]
    do = dout.reshape(B, seq_len, n_heads, head_dim).permute(0, 2, 1, 3)
    o, _ = _attn_fwd_ref(q, k, v, causal, scale)
    dq, dk, dv = _attn_bwd_ref(q, k, v, o, lse, do, causal, scale)
    if rotary_dim:
        dq = _rotary_ref(dq, sin, cos, rotary_dim, True)
        dk = _rotary_ref(dk, sin, cos, rotary_dim, True)
    return torch.cat([t.permute(0, 2, 1, 3).reshape(T, n_heads * head_dim) for t in (dq, dk, dv)],
                     dim=-1).to(qkv_rot.dtype)


def _vjp_attn_qkv(ctx, op, gs):
    qkv, sin, cos = op.inputs
    out, rot, lse = op.outputs
    a = {k: v for k, v in op.attrs.items() if k != "inplace"}
    return [emit1("attention_qkv_grad", [ctx.fwd(rot), ctx.fwd(lse), gs[0], ctx.fwd(sin), ctx.fwd(cos), ctx.fwd(out)], a),
            None, None]


def _attn_qkv_flops(op):
    a = op.attrs
    T = op.inputs[0].shape[0]
    f = 4 * T * a["seq_len"] * a["n_heads"] * a["head_dim"]
    return f // 2 if a["causal"] else f


OpDef("attention_qkv", impl=_attn_qkv_fwd_ref, vjp=_vjp_attn_qkv, flops=_attn_qkv_flops)
OpDef("attention_qkv_grad", impl=_attn_qkv_bwd_ref, flops=lambda op: int(2.5 * _attn_qkv_flops(op)))


def attention_qkv(qkv: Tensor, sin: Tensor, cos: Tensor, seq_len: int, n_heads: int, head_dim: int,
                  rotary_dim: int = 0, causal: bool = True, scale: Optional[float] = None,
                  inplace: bool = False) -> Tensor:
    """Self-attention on a packed projection `qkv (batch*seq, 3*heads*head_dim)` = `[q | k | v]`: rotary embedding of
    q and k (first `rotary_dim` features of every head, interleaved pairs; 0 disables), causal softmax attention,
    output `(batch*seq, heads*head_dim)` ready for the output projection. Heads are addressed as strided views of the
    packed matrix, so no transposes are materialised. `inplace=True` lets the kernel rotate q and k inside `qkv`."""
    if qkv.rank != 2 or qkv.shape[1] != 3 * n_heads * head_dim or qkv.shape[0] % seq_len:
        raise ValueError(f"qkv must be (batch*seq, 3*heads*head_dim); got {qkv.shape}")
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    return emit("attention_qkv", [qkv, sin, cos],
                dict(seq_len=int(seq_len), n_heads=int(n_heads), head_dim=int(head_dim), rotary_dim=int(rotary_dim),
                     causal=bool(causal), scale=scale, inplace=bool(inplace)))[0]
