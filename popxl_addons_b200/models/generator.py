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
from ..layers.embedding import Embedding
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
        self.bias = None
        if bias:
            brg = rg if bias_rg == "same" else None
            bn = brg.num_groups if brg is not None else 1
            b = np.zeros((out_f,), np.float32)
            self.bias = xl.variable(np.stack([b] * bn) if bn > 1 else b, dtype, f"{name}.bias", replica_grouping=brg)

    def tensors(self):
        d = {"weight_compressed": self.packed, "weight_decompression_scale": self.scale,
             "weight_decompression_bias": self.zero}
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
            vshard = Embedding.get_vocab_shard_size(cfg.vocab_size, cfg.tp)
            n = rg.num_groups if rg is not None else 1

            def rep(a):
                return np.stack([a] * n) if n > 1 else a

            self.wte = xl.variable(rep(np.zeros((vshard, cfg.hidden), np.float32)), dt, "wte.weight", replica_grouping=rg)
            self.ln_f = (xl.variable(np.ones(cfg.hidden, np.float32), dt, "ln_f.weight"),
                         xl.variable(np.zeros(cfg.hidden, np.float32), dt, "ln_f.bias"))
            self.head = _GQ("lm_head", vshard, cfg.hidden, self.gs, dt, rg, bias=True, scale_dtype=sdt)
            offs = Embedding.get_offsets(cfg.vocab_size, cfg.tp).astype(np.int32)
            self.vocab_offset = xl.variable(offs if cfg.tp > 1 else offs[0], xl.int32, "vocab_offset", replica_grouping=rg)
            self.layers = []
            for i in range(cfg.layers):
                L = {"ln_w": xl.variable(np.ones(cfg.hidden, np.float32), dt, f"layer{i}.ln_1.weight"),
                     "ln_b": xl.variable(np.zeros(cfg.hidden, np.float32), dt, f"layer{i}.ln_1.bias"),
                     "qkv": _GQ(f"layer{i}.attention.qkv", 3 * hd, cfg.hidden, self.gs, dt, rg, scale_dtype=sdt),
                     "out": _GQ(f"layer{i}.attention.out", cfg.hidden, hd, self.gs, dt, rg, scale_dtype=sdt),
                     "fc_in": _GQ(f"layer{i}.mlp.fc_in", F, cfg.hidden, self.gs, dt, rg, bias=True, scale_dtype=sdt),
                     "fc_out": _GQ(f"layer{i}.mlp.fc_out", cfg.hidden, F, self.gs, dt, rg, bias=True, bias_rg=None,
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

            def select_token(h, lnw, lnb, head, off):
                """Final norm, vocabulary-sharded logits, greedy choice agreed between the shards."""
                hn = ops.layer_norm(h, lnw, lnb, eps=cfg.eps)
                logits = _linear_gq(hn, head)
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

            def block(x, L, decode: bool, pos=None):
                h = ops.layer_norm(x, L["ln_w"], L["ln_b"], eps=cfg.eps)
                qkv = _linear_gq(h, L["qkv"])
                if decode:
                    qkv = ops.rotary_kv_append_(qkv, sin_tab_i, cos_tab_i, L["k"], L["v"], pos, H, D, cfg.rotary_dim)
                    a = ops.attention_decode_packed(qkv, L["k"], L["v"], pos, H, D)
                else:
                    out, rot, _ = emit("attention_qkv", [qkv, sin_p_i, cos_p_i],
                                                 dict(seq_len=P, n_heads=H, head_dim=D, rotary_dim=cfg.rotary_dim,
                                                      causal=True, scale=1.0 / float(np.sqrt(D)), inplace=True))
                    ops.kv_cache_fill_(rot, L["k"], L["v"], P, H, D)
                    a = out
                o = _linear_gq(a, L["out"])
                z = ops.gelu(_linear_gq(h, L["fc_in"]))
                y = _linear_gq(z, L["fc_out"], use_bias=False)
                y = all_reduce(o + y)
                return x + y + L["fc_out"]["bias"]

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
                for key in ("qkv", "out", "fc_in", "fc_out"):
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
                    for key in ("qkv", "out", "fc_in", "fc_out"):
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
                    x = block(x, L, decode=False)
                last = ops.reshape(x, (B, P, cfg.hidden))[:, P - 1]
                tok = select_token(last, ins["ln_f_w"], ins["ln_f_b"], head, ins["off"])
                ops.var_updates.copy_var_update_(ins["cur"], tok)
                ops.store_row_(ins["out_buf"], ins["pos"], tok, base=P)

            def decode_body(ins):
                nonlocal sin_tab_i, cos_tab_i
                sin_tab_i, cos_tab_i = ins["sin_tab"], ins["cos_tab"]
                layers, head = unpack(ins)
                x = embed(ins["cur"], ins["wte"], ins["off"])
                for L in layers:
                    x = block(x, L, decode=True, pos=ins["pos"])
                tok = select_token(x, ins["ln_f_w"], ins["ln_f_b"], head, ins["off"])
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
            for key in ("qkv", "out", "fc_in", "fc_out"):
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
        hd_full = cfg.heads * cfg.head_dim

        def shard_out(w, r, parts=1):
            # split the output rows into `parts` equal sections (q, k, v) and take rank r's slice of each
            secs = np.split(w, parts, axis=0)
            return np.concatenate([np.split(sec, tp, axis=0)[r] for sec in secs], axis=0)

        for name, q, _ in self._gq_sets():
            w = np.asarray(weights[name], np.float32)
            b = weights.get(f"{name}.bias")
            for r in range(s.num_local):
                tr = s.global_replica(r) % tp
                col_parallel = name.endswith(("qkv", "fc_in")) or name == "lm_head"
                if name == "lm_head":
                    pad = q.out_f * tp - w.shape[0]
                    wl = np.split(np.pad(w, ((0, pad), (0, 0))), tp, axis=0)[tr]
                    bl = None if b is None else np.split(np.pad(np.asarray(b, np.float32), (0, pad)), tp)[tr]
                elif col_parallel:
                    parts = 3 if name.endswith("qkv") else 1
                    wl = shard_out(w, tr, parts)
                    bl = None if b is None else shard_out(np.asarray(b, np.float32)[:, None], tr, parts)[:, 0]
                else:
                    wl = np.split(w, tp, axis=1)[tr]
                    bl = None if b is None else np.asarray(b, np.float32)
                packed, scale, zero = quantize_rows(torch.tensor(wl), self.gs)
                s._vars[q.packed][r].view(torch.int16).copy_(packed)
                s._vars[q.scale][r].copy_(scale.to(s._vars[q.scale][r].dtype))
                s._vars[q.zero][r].copy_(zero.to(s._vars[q.zero][r].dtype))
                if bl is not None and q.bias is not None:
                    s._vars[q.bias][r].copy_(torch.tensor(bl).to(s._vars[q.bias][r].dtype))
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
