"""Greedy generation with 4-bit group-quantised weights, tensor parallel over the replica set.

Every Linear of the decoder is a `LinearGQ`-format weight (groups of `group_size` along the *input* dimension, i.e.
`dim=0`: packed `(out, in/gs, gs/4)` uint16 plus per-group scale and bias in the compute dtype). Column-parallel layers
(qkv, fc_in, lm_head) shard the output rows, row-parallel layers (attention out, fc_out) shard the input columns and are
followed by an all-reduce. The program has two graphs:

* prefill: the whole prompt through the layers (de-quantise once per weight + tcgen05 GEMM, causal attention on the
  packed qkv), filling the bf16 KV cache and producing the first token;
* decode step: one token per sequence. All position-dependent ops read a device-side position, nothing in the step
  depends on the host, and the step is the body of an `ops.repeat(..., cuda_graph=True)` loop: captured once, replayed.

The reference provides the quantised layer and its decompress op (layers/linear_gq.py:19-136,
ops/group_quantize_decompress) but no generation program; this is the composition its GPT-J inference application makes.
"""
import os
from typing import Dict, Optional

import numpy as np
import torch

from .. import xl
from ..layers.embedding import Embedding, model_vocab_offsets, model_vocab_shard_size
from ..layers.linear_gq import interleave_scale_zero, linear_gq_window_t
from ..named_tensors import NamedTensors
from ..ops.group_quantize_decompress import group_quantize_compress_numpy
from ..ops.rotary_pos_embed import trig_tables
from ..streams import InputStreams, OutputStreams
from ..task_session import TaskSession
from ..xl import ops
from ..xl.opdef import emit, emit1
from .decoder import DecoderConfig, _Parallel

__all__ = ["DecoderGenerator", "quantize_rows"]


def quantize_rows(w: torch.Tensor, group_size: int = 64):
    """4-bit group quantisation of `w (out, in)` along `in` with torch ops (works on any device).
    Returns `(packed int16-view-of-uint16 (out, in/gs, gs/4), scale (out, in/gs, 1), zero (out, in/gs, 1))` where
    `value = code * scale + zero`, first element of a word in its most significant nibble."""
    out_f, in_f = w.shape
    g = w.float().reshape(out_f, in_f // group_size, group_size)
    lo = g.amin(dim=-1, keepdim=True)
    hi = g.amax(dim=-1, keepdim=True)
    scale = (hi - lo) / 15.0
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    codes = torch.clamp(torch.round((g - lo) / safe), 0, 15).to(torch.int32)
    codes = codes.reshape(out_f, in_f // group_size, group_size // 4, 4)
    packed = (codes[..., 0] << 12) | (codes[..., 1] << 8) | (codes[..., 2] << 4) | codes[..., 3]
    packed = packed.to(torch.int32)
    packed = torch.where(packed >= 32768, packed - 65536, packed).to(torch.int16)  # same bits as uint16
    return packed, scale, lo


class _GQ:
    """Variables of one quantised linear (this rank's shard)."""

    def __init__(self, name, out_f, in_f, gs, dtype, rg, bias=False, bias_rg="same", scale_dtype=None):
        self.out_f, self.in_f, self.gs = out_f, in_f, gs
        z16 = np.zeros((out_f, in_f // gs, gs // 4), np.uint16)
        n = rg.num_groups if rg is not None else 1

        def rep(a):
            return np.stack([a] * n) if n > 1 else a

        self.packed = xl.variable(rep(z16), xl.uint16, f"{name}.weight_compressed", replica_grouping=rg)
        ones = np.ones((out_f, in_f // gs, 1), np.float32)
        sdt = scale_dtype or dtype
        self.scale = xl.variable(rep(ones), sdt, f"{name}.weight_decompression_scale", replica_grouping=rg)
        self.zero = xl.variable(rep(0 * ones), sdt, f"{name}.weight_decompression_bias", replica_grouping=rg)
        # the same scales and zero points as (scale, zero) pairs, group-major: the layout the decode kernel reads
        self.sz = xl.variable(rep(np.zeros((in_f // gs, out_f, 2), np.float32)), sdt, f"{name}.weight_scale_zero_t",
                              replica_grouping=rg)
        self.bias = None
        if bias:
            brg = rg if bias_rg == "same" else None
            bn = brg.num_groups if brg is not None else 1
            b = np.zeros((out_f,), np.float32)
            self.bias = xl.variable(np.stack([b] * bn) if bn > 1 else b, dtype, f"{name}.bias", replica_grouping=brg)

    def tensors(self):
        d = {"weight_compressed": self.packed, "weight_decompression_scale": self.scale,
             "weight_decompression_bias": self.zero, "weight_scale_zero_t": self.sz}
        if self.bias is not None:
            d["bias"] = self.bias
        return d


def _linear_gq(x, w: Dict[str, xl.Tensor], use_bias=True):
    ins = [x, w["weight_compressed"], w["weight_decompression_scale"], w["weight_decompression_bias"]]
    if use_bias and "bias" in w:
        ins.append(w["bias"])
    return emit1("linear_gq", ins, {"dim": 0})


class DecoderGenerator:
    def __init__(self, cfg: DecoderConfig, batch: int = 16, prompt_len: int = 512, max_new_tokens: int = 128,
                 group_size: int = 64, device: str = "auto", seed: int = 0, cuda_graphs: bool = True,
                 use_native: Optional[bool] = None, scale_dtype: Optional[xl.dtype] = None):
        """`scale_dtype`: type of the per-group scale and bias (default: fp16 for 16-bit models, as the reference's
        LinearGQ stores them; the model dtype otherwise)."""
        if cfg.family != "gptj":
            raise NotImplementedError("the generation program is written for the GPT-J block layout")
        if cfg.dp != 1:
            raise ValueError("generation uses tensor parallelism only (dp must be 1)")
        from ..layers import linear_gq as _register_linear_gq  # noqa: F401  (defines the linear_gq op)

        self.cfg, self.batch, self.prompt_len, self.max_new, self.gs = cfg, batch, prompt_len, max_new_tokens, group_size
        self.max_seq = prompt_len + max_new_tokens
        self.scale_dtype = scale_dtype or (xl.float16 if cfg.xl_dtype in (xl.float16, xl.bfloat16) else cfg.xl_dtype)
        world = int(os.environ.get("WORLD_SIZE", "1"))
        self.ir = xl.Ir(replication="popdist" if world > 1 else cfg.tp)
        self.cuda_graphs = cuda_graphs
        self._build()
        self.session = TaskSession(self.inputs, self.outputs, self.state, 1, self.ir, device, use_native=use_native)
        self._init_weights(seed)

    # ------------------------------------------------------------------------------------------------------------
    def _build(self):
        cfg, ir = self.cfg, self.ir
        B, P, S = self.batch, self.prompt_len, self.max_seq
        dt, sdt = cfg.xl_dtype, self.scale_dtype
        H = cfg.heads // cfg.tp
        D, hd = cfg.head_dim, (cfg.heads // cfg.tp) * cfg.head_dim
        F = cfg.ffn // cfg.tp
        with ir.main_graph:
            par = _Parallel(cfg)
            rg = par.sharded_rg
            tp_group = par.tp_group
            self.inputs = InputStreams(prompt=((B, P), xl.int32))
            self.outputs = OutputStreams(tokens=((self.max_new, B), xl.int32))
            sin_np, cos_np = trig_tables(S, cfg.rotary_dim)
            sin_tab, cos_tab = xl.constant(sin_np, dt, "sin_table"), xl.constant(cos_np, dt, "cos_table")
            sin_p, cos_p = xl.constant(sin_np[None, :P], dt, "sin_prompt"), xl.constant(cos_np[None, :P], dt, "cos_prompt")
            vshard = model_vocab_shard_size(cfg.vocab_size, cfg.tp)
            n = rg.num_groups if rg is not None else 1

            def rep(a):
                return np.stack([a] * n) if n > 1 else a

            self.wte = xl.variable(rep(np.zeros((vshard, cfg.hidden), np.float32)), dt, "wte.weight", replica_grouping=rg)
            self.ln_f = (xl.variable(np.ones(cfg.hidden, np.float32), dt, "ln_f.weight"),
                         xl.variable(np.zeros(cfg.hidden, np.float32), dt, "ln_f.bias"))
            self.head = _GQ("lm_head", vshard, cfg.hidden, self.gs, dt, rg, bias=True, scale_dtype=sdt)
            offs = model_vocab_offsets(cfg.vocab_size, cfg.tp).astype(np.int32)
            self.vocab_offset = xl.variable(offs if cfg.tp > 1 else offs[0], xl.int32, "vocab_offset", replica_grouping=rg)
            self.layers = []
            for i in range(cfg.layers):
                L = {"ln_w": xl.variable(np.ones(cfg.hidden, np.float32), dt, f"layer{i}.ln_1.weight"),
                     "ln_b": xl.variable(np.zeros(cfg.hidden, np.float32), dt, f"layer{i}.ln_1.bias"),
                     # both layers that read the normalised input share one weight: rows [q | k | v | fc_in]
                     "w1": _GQ(f"layer{i}.qkv_fc_in", 3 * hd + F, cfg.hidden, self.gs, dt, rg, bias=True,
                               scale_dtype=sdt),
                     # both layers whose outputs are summed share one weight: input columns [attention | fc_in output]
                     "w2": _GQ(f"layer{i}.out_fc_out", cfg.hidden, hd + F, self.gs, dt, rg, bias=True, bias_rg=None,
                               scale_dtype=sdt),
                     "k": xl.variable(np.zeros((B, H, S, D), np.float32), dt, f"layer{i}.k_cache"),
                     "v": xl.variable(np.zeros((B, H, S, D), np.float32), dt, f"layer{i}.v_cache")}
                self.layers.append(L)
            self.pos = xl.variable(np.array(P, np.int32), xl.int32, "position")
            self.cur = xl.variable(np.zeros((B,), np.int32), xl.int32, "current_token")
            self.out_buf = xl.variable(np.zeros((self.max_new, B), np.int32), xl.int32, "generated")

            def all_reduce(t):
                return ops.collectives.replicated_all_reduce(t, "add", tp_group) if cfg.tp > 1 else t

            def embed(tokens, wte, off):
                idx = tokens - off if cfg.tp > 1 else tokens
                return all_reduce(ops.gather(wte, idx, axis=0, zero_OOR=cfg.tp > 1))

            def select_token(hn, head, off):
                """Vocabulary-sharded logits of the normalised hidden state, greedy choice agreed between the shards."""
                logits = linear_gq_window_t(hn, head["weight_compressed"], head["weight_scale_zero_t"], head["bias"])
                valid = vshard  # padded rows of the last shard are excluded below via the index check
                m, idx = ops.argmax_rows(logits, valid, 0)
                idx = idx + off if cfg.tp > 1 else idx
                if cfg.tp == 1:
                    return idx
                # rows beyond the true vocabulary can only win if their (zero-weight) logit beats everything: mask them
                in_vocab = ops.cast(ops.less(idx, xl.constant(cfg.vocab_size, xl.int32)), xl.float32)
                m = m * in_vocab + (in_vocab - 1.0) * 1e30
                gmax = ops.collectives.replicated_all_reduce(m, "max", tp_group)
                cand = ops.where(ops.greater_equal(m, gmax), ops.cast(idx, xl.float32),
                                 xl.constant(float(2 ** 24), xl.float32))
                # smallest candidate index over the group = max of the negated candidates
                win = ops.negate(ops.collectives.replicated_all_reduce(ops.negate(cand), "max", tp_group))
                return ops.cast(win, xl.int32)

            def rows(w: Dict[str, xl.Tensor], lo: int, hi: int) -> Dict[str, xl.Tensor]:
                """Output rows [lo, hi) of a quantised weight (a contiguous slice of every one of its tensors)."""
                return {k: v[lo:hi] for k, v in w.items()}

            def prefill_block(x, L):
                """Whole prompt: de-quantise + tcgen05 GEMMs, causal attention on the packed projections."""
                h = ops.layer_norm(x, L["ln_w"], L["ln_b"], eps=cfg.eps)
                qkv = _linear_gq(h, rows(L["w1"], 0, 3 * hd), use_bias=False)
                out, rot, _ = emit("attention_qkv", [qkv, sin_p_i, cos_p_i],
                                   dict(seq_len=P, n_heads=H, head_dim=D, rotary_dim=cfg.rotary_dim, causal=True,
                                        scale=1.0 / float(np.sqrt(D)), inplace=True))
                ops.kv_cache_fill_(rot, L["k"], L["v"], P, H, D)
                z = ops.gelu(_linear_gq(h, rows(L["w1"], 3 * hd, 3 * hd + F)))
                y = _linear_gq(ops.concat([out, z], axis=1), L["w2"], use_bias=False)
                return x + all_reduce(y) + L["w2"]["bias"]

            def residual_norm(x, delta, delta_bias, lnw, lnb):
                """`x += all_reduce(delta) + bias; LayerNorm(x)`: one kernel, the all-reduce over the TP group included."""
                if delta is not None and cfg.tp > 1:
                    return ops.all_reduce_add_layer_norm_(x, delta, delta_bias, lnw, lnb, tp_group, eps=cfg.eps)
                return ops.add_layer_norm_(x, delta, delta_bias, lnw, lnb, eps=cfg.eps)

            def decode_block(x, delta, delta_bias, L, pos):
                """One token per sequence, five kernels: (all-reduce +) residual + LayerNorm; [qkv | gelu(fc_in)] in one
                de-quantising GEMM; rotary + cache append; attention, written next to the fc_in output; [out | fc_out] in
                one GEMM. Returns this rank's partial layer output; the next layer's first kernel reduces it."""
                h = residual_norm(x, delta, delta_bias, L["ln_w"], L["ln_b"])
                w1 = L["w1"]
                buf = linear_gq_window_t(h, w1["weight_compressed"], w1["weight_scale_zero_t"], w1["bias"],
                                         act_from_col=3 * hd)
                buf = ops.rotary_kv_append_(buf, sin_tab_i, cos_tab_i, L["k"], L["v"], pos, H, D, cfg.rotary_dim)
                buf = ops.attention_decode_into_(buf, L["k"], L["v"], pos, H, D, out_col=2 * hd)
                w2 = L["w2"]
                return linear_gq_window_t(buf, w2["weight_compressed"], w2["weight_scale_zero_t"], None, x_col=2 * hd,
                                          k=hd + F)

            # graphs take every variable as an input; collect them in a fixed order
            flat: Dict[str, xl.Tensor] = {"wte": self.wte, "ln_f_w": self.ln_f[0], "ln_f_b": self.ln_f[1],
                                          "off": self.vocab_offset, "pos": self.pos, "cur": self.cur,
                                          "out_buf": self.out_buf, "sin_tab": sin_tab, "cos_tab": cos_tab,
                                          "sin_p": sin_p, "cos_p": cos_p}
            for k, v in self.head.tensors().items():
                flat[f"head.{k}"] = v
            for i, L in enumerate(self.layers):
                for key in ("ln_w", "ln_b", "k", "v"):
                    flat[f"l{i}.{key}"] = L[key]
                for key in ("w1", "w2"):
                    for k, v in L[key].tensors().items():
                        flat[f"l{i}.{key}.{k}"] = v
            by_ref = {"pos", "cur", "out_buf"} | {f"l{i}.{k}" for i in range(cfg.layers) for k in ("k", "v")}

            def make_graph(name, body):
                g = ir.create_empty_graph(name)
                with g:
                    ins = {k: xl.graph_input(v.shape, v.dtype, k.replace(".", "_"), by_ref=k in by_ref)
                           for k, v in flat.items()}
                    body(ins)
                return g, {ins[k]: flat[k] for k in flat}

            def unpack(ins):
                layers = []
                for i in range(cfg.layers):
                    L = {key: ins[f"l{i}.{key}"] for key in ("ln_w", "ln_b", "k", "v")}
                    for key in ("w1", "w2"):
                        L[key] = {k[len(f"l{i}.{key}."):]: t for k, t in ins.items() if k.startswith(f"l{i}.{key}.")}
                    layers.append(L)
                head = {k[len("head."):]: t for k, t in ins.items() if k.startswith("head.")}
                return layers, head

            sin_tab_i = cos_tab_i = sin_p_i = cos_p_i = None

            def prefill_body(ins):
                nonlocal sin_p_i, cos_p_i
                sin_p_i, cos_p_i = ins["sin_p"], ins["cos_p"]
                layers, head = unpack(ins)
                prompt = ops.host_load(self.inputs.prompt)
                x = embed(ops.reshape(prompt, (B * P,)), ins["wte"], ins["off"])
                for L in layers:
                    x = prefill_block(x, L)
                last = ops.reshape(x, (B, P, cfg.hidden))[:, P - 1]
                hn = ops.layer_norm(last, ins["ln_f_w"], ins["ln_f_b"], eps=cfg.eps)
                tok = select_token(hn, head, ins["off"])
                ops.var_updates.copy_var_update_(ins["cur"], tok)
                ops.store_row_(ins["out_buf"], ins["pos"], tok, base=P)

            def decode_body(ins):
                nonlocal sin_tab_i, cos_tab_i
                sin_tab_i, cos_tab_i = ins["sin_tab"], ins["cos_tab"]
                layers, head = unpack(ins)
                x = embed(ins["cur"], ins["wte"], ins["off"])
                delta = delta_bias = None
                for L in layers:
                    delta = decode_block(x, delta, delta_bias, L, ins["pos"])
                    delta_bias = L["w2"]["bias"]
                hn = residual_norm(x, delta, delta_bias, ins["ln_f_w"], ins["ln_f_b"])
                tok = select_token(hn, head, ins["off"])
                ops.advance_position_(ins["pos"])
                ops.var_updates.copy_var_update_(ins["cur"], tok)
                ops.store_row_(ins["out_buf"], ins["pos"], tok, base=P)

            prefill, pre_map = make_graph("prefill", prefill_body)
            decode, dec_map = make_graph("decode_step", decode_body)
            # program: reset position, prefill, timed decode loop, read the tokens back
            ops.var_updates.copy_var_update_(self.pos, xl.constant(np.array(P, np.int32), xl.int32))
            ops.timestamp("start")
            ops.call(prefill, inputs_dict=pre_map)
            ops.timestamp("prefill_done")
            ops.repeat(decode, self.max_new - 1, inputs_dict=dec_map, cuda_graph=self.cuda_graphs)
            ops.timestamp("decode_done")
            ops.host_store(self.outputs.tokens, self.out_buf)
        from ..patterns import apply_pre_alias_patterns

        apply_pre_alias_patterns(ir)
        self.state = NamedTensors.from_dict({k.replace(".", "_"): v for k, v in flat.items()
                                             if isinstance(v, xl.Variable) and not k.endswith((".k", ".v"))})

    # ------------------------------------------------------------------------------------------------------------
    def _gq_sets(self):
        out = [("lm_head", self.head, 0)]
        for i, L in enumerate(self.layers):
            for key in ("w1", "w2"):
                out.append((f"layer{i}.{key}", L[key], i + 1))
        return out

    def _init_weights(self, seed: int):
        """Random N(0, 0.02) dense weights, drawn and quantised on the session's device, written into this rank's
        (or, in the in-process simulation, every replica's) variables."""
        s = self.session
        dev = s.device
        for name, q, salt in self._gq_sets():
            for r in range(s.num_local):
                grp = q.packed.replica_grouping.group_index(s.global_replica(r))
                gen = torch.Generator(device=dev).manual_seed(seed * 7919 + hash(name) % 100003 + 31 * grp)
                w = torch.empty((q.out_f, q.in_f), dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=gen)
                packed, scale, zero = quantize_rows(w, self.gs)
                s._vars[q.packed][r].view(torch.int16).copy_(packed)
                s._vars[q.scale][r].copy_(scale.to(s._vars[q.scale][r].dtype))
                s._vars[q.zero][r].copy_(zero.to(s._vars[q.zero][r].dtype))
                s._vars[q.sz][r].copy_(interleave_scale_zero(s._vars[q.scale][r], s._vars[q.zero][r]))
        for r in range(s.num_local):
            grp = self.wte.replica_grouping.group_index(s.global_replica(r))
            gen = torch.Generator(device=dev).manual_seed(seed * 7919 + 17 + grp)
            t = s._vars[self.wte][r]
            t.copy_(torch.empty(t.shape, dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=gen).to(t.dtype))

    def load_dense(self, weights: Dict[str, np.ndarray]):
        """Quantise and shard full (un-sharded) dense weights given as `{name: (out, in) array}` for the linears
        (`lm_head`, `layer{i}.qkv|out|fc_in|fc_out`, optional `<name>.bias`), `wte`, `ln_f.weight/bias`,
        `layer{i}.ln_1.weight/bias`. qkv rows are ordered `[q | k | v]`, each head-major."""
        cfg, tp = self.cfg, self.cfg.tp
        s = self.session

        def f32(name):
            v = weights.get(name)
            return None if v is None else np.asarray(v, np.float32)

        def shard_rows(w, r, parts=1):
            # split the output rows into `parts` equal sections (q, k, v) and take rank r's slice of each
            secs = np.split(w, parts, axis=0)
            return np.concatenate([np.split(sec, tp, axis=0)[r] for sec in secs], axis=0)

        def store(q, r, wl, bl):
            packed, scale, zero = quantize_rows(torch.tensor(wl), self.gs)
            s._vars[q.packed][r].view(torch.int16).copy_(packed)
            s._vars[q.scale][r].copy_(scale.to(s._vars[q.scale][r].dtype))
            s._vars[q.zero][r].copy_(zero.to(s._vars[q.zero][r].dtype))
            s._vars[q.sz][r].copy_(interleave_scale_zero(s._vars[q.scale][r], s._vars[q.zero][r]))
            if bl is not None and q.bias is not None:
                s._vars[q.bias][r].copy_(torch.tensor(bl).to(s._vars[q.bias][r].dtype))

        for r in range(s.num_local):
            tr = s.global_replica(r) % tp
            w, b = f32("lm_head"), f32("lm_head.bias")
            pad = self.head.out_f * tp - w.shape[0]
            store(self.head, r, np.split(np.pad(w, ((0, pad), (0, 0))), tp, axis=0)[tr],
                  None if b is None else np.split(np.pad(b, (0, pad)), tp)[tr])
            for i, L in enumerate(self.layers):
                qkv, fc_in = f32(f"layer{i}.qkv"), f32(f"layer{i}.fc_in")
                qkv_l, fc_in_l = shard_rows(qkv, tr, 3), shard_rows(fc_in, tr)
                b_qkv, b_fc = f32(f"layer{i}.qkv.bias"), f32(f"layer{i}.fc_in.bias")
                b1 = np.concatenate([
                    np.zeros(qkv_l.shape[0], np.float32) if b_qkv is None else shard_rows(b_qkv[:, None], tr, 3)[:, 0],
                    np.zeros(fc_in_l.shape[0], np.float32) if b_fc is None else shard_rows(b_fc[:, None], tr)[:, 0]])
                store(L["w1"], r, np.concatenate([qkv_l, fc_in_l], axis=0), b1)
                out_l = np.split(f32(f"layer{i}.out"), tp, axis=1)[tr]
                fc_out_l = np.split(f32(f"layer{i}.fc_out"), tp, axis=1)[tr]
                b_out, b_fco = f32(f"layer{i}.out.bias"), f32(f"layer{i}.fc_out.bias")
                b2 = np.zeros(cfg.hidden, np.float32)
                for bb in (b_out, b_fco):
                    if bb is not None:
                        b2 = b2 + bb
                store(L["w2"], r, np.concatenate([out_l, fc_out_l], axis=1), b2)
        vshard = self.wte.shape[0]
        wte = np.asarray(weights["wte"], np.float32)
        wte = np.pad(wte, ((0, vshard * tp - wte.shape[0]), (0, 0)))
        for r in range(s.num_local):
            tr = s.global_replica(r) % tp
            s._vars[self.wte][r].copy_(torch.tensor(np.split(wte, tp)[tr]).to(s._vars[self.wte][r].dtype))
            for var, key in ((self.ln_f[0], "ln_f.weight"), (self.ln_f[1], "ln_f.bias")):
                if key in weights:
                    s._vars[var][r].copy_(torch.tensor(np.asarray(weights[key], np.float32)).to(s._vars[var][r].dtype))
            for i, L in enumerate(self.layers):
                for var, key in ((L["ln_w"], f"layer{i}.ln_1.weight"), (L["ln_b"], f"layer{i}.ln_1.bias")):
                    if key in weights:
                        s._vars[var][r].copy_(torch.tensor(np.asarray(weights[key], np.float32)).to(
                            s._vars[var][r].dtype))

    # ------------------------------------------------------------------------------------------------------------
    def generate(self, prompt) -> np.ndarray:
        """`prompt`: int32 `(batch, prompt_len)` (identical on all ranks). Returns `(batch, max_new_tokens)` int32."""
        if not isinstance(prompt, torch.Tensor):  # tensors (e.g. pinned host memory) are handed through as they are
            prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        if self.session.num_local > 1:
            prompt = np.stack([np.asarray(prompt)] * self.session.num_local)
        out = self.session.run({self.inputs.prompt: prompt})[self.outputs.tokens]
        out = np.asarray(out)
        if out.ndim == 3:  # in-process simulation: one copy per replica, all identical
            out = out[0]
        return out.T.copy()

    def decode_ms(self) -> float:
        return self.session.elapsed_ms("prefill_done", "decode_done")

    def prefill_ms(self) -> float:
        return self.session.elapsed_ms("start", "prefill_done")
