"""Decoder-only transformer family (GPT-2, GPT-J, Llama shapes) written as add-on Modules.

The reference ships building blocks only; its users (Graphcore's GPT-J / GPT-3 / Llama applications) assemble models
like these from `Linear`, `LayerNorm`, `Embedding`, the tensor-parallel all-reduce pair, the vocabulary-sharded
cross-entropy and the rotary op. The assembly here follows the same recipe: tensor-parallel shards are declared through
the *data-parallel* replica grouping (identical across DP, different across TP), column-parallel layers are preceded by
the forward-identity all-reduce and row-parallel layers are followed by the backward-identity all-reduce
(tests/integration/test_batch_serialisation.py:463-492 of popxl_addons shows the pattern on a feed-forward block).
"""
import math
from dataclasses import dataclass, replace
from typing import Optional

import numpy as np

from .. import xl
from ..layers.embedding import Embedding, model_vocab_offsets, model_vocab_shard_size
from ..module import Module
from ..ops.cross_entropy_sharded_loss import cross_entropy_sharded_loss
from ..ops.replicated_all_reduce_TP import (replicated_all_reduce_identical_grad_inputs,
                                            replicated_all_reduce_identical_inputs)
from ..ops.rotary_pos_embed import trig_tables
from ..xl import ops

__all__ = ["DecoderConfig", "DecoderBlock", "DecoderEmbedding", "DecoderHead"]


@dataclass
class DecoderConfig:
    family: str = "gptj"            # "gptj" | "gpt2" | "llama"
    layers: int = 28
    hidden: int = 4096
    heads: int = 16
    head_dim: int = 256
    rotary_dim: int = 64
    ffn: int = 16384
    vocab_size: int = 50400
    seq_len: int = 2048
    eps: float = 1e-5
    dtype: str = "bfloat16"
    init_std: float = 0.02
    tp: int = 1
    dp: int = 1
    # Sequence parallelism inside the TP group: the residual stream, the norms and the residual adds work on
    # `tokens / tp` rows per rank; the TP all-reduces become reduce-scatter (after the row-parallel linears) and
    # all-gather (before the column-parallel ones): same bytes on the wire, 1/tp of the elementwise work.
    sequence_parallel: bool = False

    @property
    def sp(self) -> bool:
        return self.sequence_parallel and self.tp > 1

    @property
    def xl_dtype(self) -> xl.dtype:
        return xl.dtype.as_dtype(self.dtype)

    @property
    def np_dtype(self):
        return np.float32 if self.dtype in ("bfloat16", "float32") else np.float16

    def with_parallelism(self, tp: int, dp: int) -> "DecoderConfig":
        return replace(self, tp=tp, dp=dp)

    def param_count(self) -> int:
        h, f = self.hidden, self.ffn
        attn = 4 * h * self.heads * self.head_dim
        mlp = (3 if self.family == "llama" else 2) * h * f
        emb = self.vocab_size * h * (1 if self.family == "gpt2" else 2)
        return self.layers * (attn + mlp) + emb

    # -- named shapes --------------------------------------------------------------------------------------------
    @classmethod
    def gptj_6b(cls, **kw):
        return cls(family="gptj", layers=28, hidden=4096, heads=16, head_dim=256, rotary_dim=64, ffn=16384,
                   vocab_size=50400, seq_len=2048, **kw)

    @classmethod
    def gpt2_small(cls, **kw):
        return cls(family="gpt2", layers=12, hidden=768, heads=12, head_dim=64, rotary_dim=0, ffn=3072,
                   vocab_size=50257, seq_len=1024, **kw)

    @classmethod
    def llama2_7b(cls, **kw):
        return cls(family="llama", layers=32, hidden=4096, heads=32, head_dim=128, rotary_dim=128, ffn=11008,
                   vocab_size=32000, seq_len=2048, **kw)

    @classmethod
    def tiny(cls, family: str = "gptj", **kw):
        base = dict(family=family, layers=2, hidden=128, heads=4, head_dim=32, rotary_dim=16 if family != "gpt2" else 0,
                    ffn=256, vocab_size=512, seq_len=64)
        base.update(kw)
        return cls(**base)


_SEED = [0]


def _normal(shape, std, np_dtype):
    """Factory data source: a recipe that the session materialises on the device (a fresh seed per draw)."""

    def draw():
        _SEED[0] += 1
        return xl.LazyInit(shape, np_dtype, "normal", std, seed=_SEED[0])

    return draw


def _const_init(kind, shape, np_dtype):
    return lambda: xl.LazyInit(shape, np_dtype, kind)


class _Parallel:
    """Replica groupings of a TP x DP layout: TP ranks are consecutive replicas."""

    def __init__(self, cfg: DecoderConfig):
        ir = xl.gcg().ir
        self.tp, self.dp = cfg.tp, cfg.dp
        if cfg.tp * cfg.dp != ir.replication_factor:
            raise ValueError(f"tp*dp = {cfg.tp * cfg.dp} must equal the replication factor {ir.replication_factor}")
        self.tp_group = ir.replica_grouping(stride=1, group_size=cfg.tp)
        self.dp_group = ir.replica_grouping(stride=cfg.tp, group_size=cfg.dp)
        self.all = ir.replica_grouping()

    @property
    def sharded_rg(self):
        """Grouping for a tensor-parallel shard: identical across DP."""
        return self.dp_group if self.tp > 1 else None


def _gather_tokens(h_s: xl.Tensor, par: "_Parallel") -> xl.Tensor:
    """`(tokens/tp, hidden)` rows of every TP rank -> `(tokens, hidden)`; gradient: reduce-scatter."""
    rows, hidden = h_s.shape
    return ops.collectives.replicated_all_gather(h_s, par.tp_group, output_shape=(rows * par.tp, hidden))


def _scatter_tokens(s: xl.Tensor, par: "_Parallel") -> xl.Tensor:
    """Sum of the ranks' partial `(tokens, hidden)` results, this rank's `tokens/tp` rows; gradient: all-gather."""
    rows, hidden = s.shape
    if rows % par.tp:
        raise ValueError(f"sequence parallelism needs the token count ({rows}) to be a multiple of tp={par.tp}")
    return ops.reshape(ops.collectives.replicated_reduce_scatter(s, "add", par.tp_group), (rows // par.tp, hidden))


class DecoderBlock(Module):
    """One transformer layer on `(tokens, hidden)` activations (tokens = micro_batch * seq_len)."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg

    def _linear(self, name, x, out_features, bias, par, std=None):
        cfg = self.cfg
        w = self.add_variable_input(f"{name}.weight", _normal((x.shape[-1], out_features), std or cfg.init_std,
                                                              cfg.np_dtype), cfg.xl_dtype,
                                    replica_grouping=par.sharded_rg, overwrite=True)
        b = None
        if bias:
            b = self.add_variable_input(f"{name}.bias", _const_init("zeros", (out_features,), cfg.np_dtype), cfg.xl_dtype,
                                        replica_grouping=par.sharded_rg, overwrite=True)
        return w, b

    def _norm(self, name, x):
        cfg = self.cfg
        w = self.add_variable_input(f"{name}.weight", _const_init("ones", (cfg.hidden,), cfg.np_dtype), cfg.xl_dtype,
                                    overwrite=True)
        if cfg.family == "llama":
            return ops.rms_norm(x, w, eps=cfg.eps)
        b = self.add_variable_input(f"{name}.bias", _const_init("zeros", (cfg.hidden,), cfg.np_dtype), cfg.xl_dtype,
                                    overwrite=True)
        return ops.layer_norm(x, w, b, eps=cfg.eps)

    def _attention(self, h, sin, cos, par, collectives: bool = True):
        """`collectives=False`: the caller has marked `h` as identical over the TP group and reduces the result itself
        (blocks whose attention and feed-forward share input and output need one all-reduce, not two)."""
        cfg = self.cfg
        heads = cfg.heads // par.tp
        hd = heads * cfg.head_dim
        bias = cfg.family == "gpt2"
        if par.tp > 1 and collectives:
            h = replicated_all_reduce_identical_inputs(h, group=par.tp_group)
        wqkv, bqkv = self._linear("attention.qkv", h, 3 * hd, bias, par)
        qkv = ops.linear_bias_act(h, wqkv, bqkv) if bqkv is not None else h @ wqkv
        a = ops.attention_qkv(qkv, sin, cos, cfg.seq_len, heads, cfg.head_dim, cfg.rotary_dim, causal=True,
                              inplace=True)
        wo = self.add_variable_input("attention.out.weight",
                                     _normal((hd, cfg.hidden), cfg.init_std / math.sqrt(2 * cfg.layers), cfg.np_dtype),
                                     cfg.xl_dtype, replica_grouping=par.sharded_rg, overwrite=True)
        o = a @ wo
        if par.tp > 1 and collectives:
            o = replicated_all_reduce_identical_grad_inputs(o, group=par.tp_group)
        bo = None
        if bias:
            bo = self.add_variable_input("attention.out.bias", _const_init("zeros", (cfg.hidden,), cfg.np_dtype),
                                         cfg.xl_dtype, overwrite=True)
        if not collectives:
            return o, bo  # partial result: the caller reduces it and adds the bias once
        return o + bo if bo is not None else o

    def _mlp(self, h, par, collectives: bool = True):
        """With `collectives=False` returns `(partial result, output bias)`: the caller reduces and adds the bias."""
        cfg = self.cfg
        f = cfg.ffn // par.tp
        if par.tp > 1 and collectives:
            h = replicated_all_reduce_identical_inputs(h, group=par.tp_group)
        if cfg.family == "llama":
            wg, _ = self._linear("mlp.gate", h, f, False, par)
            wu, _ = self._linear("mlp.up", h, f, False, par)
            z = ops.swiglu(h @ wg, h @ wu)
        else:
            w1, b1 = self._linear("mlp.fc_in", h, f, True, par)
            # the bias is added in the GEMM epilogue; the activation stays a separate op because its input is needed
            # again by the backward pass
            z = ops.gelu(ops.linear_bias_act(h, w1, b1), approximate="tanh" if cfg.family == "gpt2" else "none")
        w2 = self.add_variable_input("mlp.fc_out.weight",
                                     _normal((f, cfg.hidden), cfg.init_std / math.sqrt(2 * cfg.layers), cfg.np_dtype),
                                     cfg.xl_dtype, replica_grouping=par.sharded_rg, overwrite=True)
        b2 = None
        if cfg.family != "llama":
            b2 = self.add_variable_input("mlp.fc_out.bias", _const_init("zeros", (cfg.hidden,), cfg.np_dtype),
                                         cfg.xl_dtype, overwrite=True)
        if not collectives:
            return z @ w2, b2
        if par.tp == 1 and b2 is not None:
            return ops.linear_bias_act(z, w2, b2)
        y = z @ w2
        if par.tp > 1:
            y = replicated_all_reduce_identical_grad_inputs(y, group=par.tp_group)
        return y + b2 if b2 is not None else y

    def build(self, x: xl.Tensor, sin: xl.Tensor, cos: xl.Tensor) -> xl.Tensor:
        cfg = self.cfg
        par = _Parallel(cfg)
        if cfg.sp:
            # x holds this rank's tokens/tp rows; gather before the column-parallel linears, scatter after the
            # row-parallel ones
            if cfg.family == "gptj":
                h = _gather_tokens(self._norm("ln_1", x), par)
                o, _ = self._attention(h, sin, cos, par, collectives=False)
                y, b2 = self._mlp(h, par, collectives=False)
                return x + _scatter_tokens(o + y, par) + b2
            h = _gather_tokens(self._norm("ln_1", x), par)
            o, bo = self._attention(h, sin, cos, par, collectives=False)
            x = x + _scatter_tokens(o, par)
            if bo is not None:
                x = x + bo
            h = _gather_tokens(self._norm("ln_2", x), par)
            y, b2 = self._mlp(h, par, collectives=False)
            x = x + _scatter_tokens(y, par)
            return x + b2 if b2 is not None else x
        if cfg.family == "gptj":
            # parallel residual: attention and feed-forward read the same normalised input
            h = self._norm("ln_1", x)
            if par.tp == 1:
                return x + self._attention(h, sin, cos, par) + self._mlp(h, par)
            # one identity / all-reduce pair around both branches: a single all-reduce per layer in the forward pass
            # (of the summed partial results) and a single one in the backward pass (of the summed input gradients)
            h = replicated_all_reduce_identical_inputs(h, group=par.tp_group)
            o, _ = self._attention(h, sin, cos, par, collectives=False)
            y, b2 = self._mlp(h, par, collectives=False)
            s = replicated_all_reduce_identical_grad_inputs(o + y, group=par.tp_group)
            return x + s + b2
        x = x + self._attention(self._norm("ln_1", x), sin, cos, par)
        return x + self._mlp(self._norm("ln_2", x), par)


class DecoderEmbedding(Module):
    """Token (and for GPT-2 learned position) embedding with the vocabulary sharded over the TP group."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg

    def build(self, tokens: xl.Tensor, shard_offset: Optional[xl.Tensor] = None) -> xl.Tensor:
        cfg = self.cfg
        par = _Parallel(cfg)
        shard = model_vocab_shard_size(cfg.vocab_size, par.tp)
        w = self.add_variable_input("wte.weight", _normal((shard, cfg.hidden), cfg.init_std, cfg.np_dtype),
                                    cfg.xl_dtype, replica_grouping=par.sharded_rg, overwrite=True)
        idx = tokens if shard_offset is None else tokens - shard_offset
        x = ops.gather(w, idx, axis=0, zero_OOR=par.tp > 1)
        if cfg.sp:
            if cfg.family == "gpt2":
                # learned positions: every rank adds 1/tp of them to its partial lookup, the scatter sums them up
                wpe = self.add_variable_input("wpe.weight",
                                              _normal((cfg.seq_len, cfg.hidden), cfg.init_std, cfg.np_dtype),
                                              cfg.xl_dtype, overwrite=True)
                reps = tokens.shape[0] // cfg.seq_len
                pos = wpe if reps == 1 else ops.tile(wpe, (reps, 1))
                x = x + pos * (1.0 / par.tp)
            return _scatter_tokens(x, par)
        if par.tp > 1:
            x = replicated_all_reduce_identical_grad_inputs(x, group=par.tp_group)
        if cfg.family == "gpt2":
            wpe = self.add_variable_input("wpe.weight", _normal((cfg.seq_len, cfg.hidden), cfg.init_std, cfg.np_dtype),
                                          cfg.xl_dtype, overwrite=True)
            reps = tokens.shape[0] // cfg.seq_len
            pos = wpe if reps == 1 else ops.tile(wpe, (reps, 1))
            x = x + pos
        return x


class DecoderHead(Module):
    """Final norm + LM head producing this rank's slice of the logits."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg

    def build(self, x: xl.Tensor) -> xl.Tensor:
        cfg = self.cfg
        par = _Parallel(cfg)
        w = self.add_variable_input("ln_f.weight", _const_init("ones", (cfg.hidden,), cfg.np_dtype), cfg.xl_dtype,
                                    overwrite=True)
        if cfg.family == "llama":
            h = ops.rms_norm(x, w, eps=cfg.eps)
        else:
            b = self.add_variable_input("ln_f.bias", _const_init("zeros", (cfg.hidden,), cfg.np_dtype), cfg.xl_dtype,
                                        overwrite=True)
            h = ops.layer_norm(x, w, b, eps=cfg.eps)
        if cfg.sp:
            h = _gather_tokens(h, par)
        elif par.tp > 1:
            h = replicated_all_reduce_identical_inputs(h, group=par.tp_group)
        shard = model_vocab_shard_size(cfg.vocab_size, par.tp)
        wl = self.add_variable_input("lm_head.weight", _normal((cfg.hidden, shard), cfg.init_std, cfg.np_dtype),
                                     cfg.xl_dtype, replica_grouping=par.sharded_rg, overwrite=True)
        if cfg.family == "gptj":
            bl = self.add_variable_input("lm_head.bias", _const_init("zeros", (shard,), cfg.np_dtype), cfg.xl_dtype,
                                         replica_grouping=par.sharded_rg, overwrite=True)
            return ops.linear_bias_act(h, wl, bl)
        return h @ wl


def rotary_tables(cfg: DecoderConfig):
    """`(sin, cos)` constants of shape `(1, seq_len, rotary_dim/2)` in the model dtype (dummies when rotary is off)."""
    r = cfg.rotary_dim if cfg.rotary_dim else 2
    sin, cos = trig_tables(cfg.seq_len, r)
    return xl.constant(sin[None], cfg.xl_dtype, "rotary_sin"), xl.constant(cos[None], cfg.xl_dtype, "rotary_cos")
