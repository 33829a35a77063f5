"""Plain PyTorch (+cuBLAS, SDPA, NCCL) implementation of the int4 generation benchmark: the number to match or beat on
the same machine.

Weights are stored 4-bit group-quantised (groups of 64 along the input dimension, fp16 scale and bias) as the benchmark
prescribes. PyTorch has no fused int4 GEMM, so each linear de-quantises its weight with tensor ops and calls cuBLAS — the
straightforward library composition. `cache_dense=True` instead keeps a bf16 copy of every weight (4x the memory,
no longer an int4 model at run time) and shows the upper bound of the library path. The decode step is captured in a CUDA
graph in both variants (the position is a device tensor), as any tuned PyTorch serving loop would do.
`python bench.py --mode decode --impl torch` drives it.
"""
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


def quantize(w, gs):
    o, i = w.shape
    g = w.float().reshape(o, i // gs, gs)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = (hi - lo) / 15
    codes = torch.clamp(torch.round((g - lo) / torch.where(scale == 0, torch.ones_like(scale), scale)), 0, 15)
    codes = codes.to(torch.uint8).reshape(o, i // 2, 2)
    packed = (codes[..., 0] << 4) | codes[..., 1]  # two codes per byte
    return packed, scale.half(), lo.half()


class QLinear:
    def __init__(self, out_f, in_f, gs, device, gen, bias=False, cache_dense=False):
        w = torch.empty(out_f, in_f, device=device).normal_(0, 0.02, generator=gen)
        self.packed, self.scale, self.zero = quantize(w, gs)
        self.gs, self.out_f, self.in_f = gs, out_f, in_f
        self.bias = torch.zeros(out_f, device=device, dtype=torch.bfloat16) if bias else None
        self.dense = self.dequant() if cache_dense else None

    def dequant(self):
        p = self.packed
        codes = torch.stack((p >> 4, p & 15), dim=-1).reshape(self.out_f, self.in_f // self.gs, self.gs)
        return (codes.to(torch.float16) * self.scale + self.zero).reshape(self.out_f, self.in_f).to(torch.bfloat16)

    def __call__(self, x):
        w = self.dense if self.dense is not None else self.dequant()
        return F.linear(x, w, self.bias)


def rotary(x, sin, cos, rot):
    xr, xp = x[..., :rot], x[..., rot:]
    x1, x2 = xr[..., ::2], xr[..., 1::2]
    y = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)
    return torch.cat((y, xp), dim=-1)


class TorchGenerator:
    def __init__(self, cfg, batch, prompt_len, new_tokens, group_size=64, cache_dense=False, cuda_graph=True):
        self.cfg, self.B, self.P, self.N = cfg, batch, prompt_len, new_tokens
        self.S = prompt_len + new_tokens
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        tp = self.tp = self.world
        dev = self.dev = torch.device("cuda", torch.cuda.current_device())
        gen = torch.Generator(device=dev).manual_seed(1234 + self.rank)
        h, H, D = cfg.hidden, cfg.heads // tp, cfg.head_dim
        self.H, self.D = H, D
        self.vshard = (cfg.vocab_size + tp - 1) // tp
        self.wte = torch.empty(self.vshard, h, device=dev).normal_(0, 0.02, generator=gen).bfloat16()
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append(dict(
                ln_w=torch.ones(h, device=dev, dtype=torch.bfloat16), ln_b=torch.zeros(h, device=dev, dtype=torch.bfloat16),
                qkv=QLinear(3 * H * D, h, group_size, dev, gen, cache_dense=cache_dense),
                out=QLinear(h, H * D, group_size, dev, gen, cache_dense=cache_dense),
                fc_in=QLinear(cfg.ffn // tp, h, group_size, dev, gen, bias=True, cache_dense=cache_dense),
                fc_out=QLinear(h, cfg.ffn // tp, group_size, dev, gen, cache_dense=cache_dense),
                fc_out_bias=torch.zeros(h, device=dev, dtype=torch.bfloat16),
                k=torch.zeros(batch, H, self.S, D, device=dev, dtype=torch.bfloat16),
                v=torch.zeros(batch, H, self.S, D, device=dev, dtype=torch.bfloat16)))
        self.ln_f = (torch.ones(h, device=dev, dtype=torch.bfloat16), torch.zeros(h, device=dev, dtype=torch.bfloat16))
        self.head = QLinear(self.vshard, h, group_size, dev, gen, bias=True, cache_dense=cache_dense)
        inv = 1.0 / (10000 ** (torch.arange(0, cfg.rotary_dim, 2, device=dev).float() / cfg.rotary_dim))
        ang = torch.arange(self.S, device=dev).float()[:, None] * inv[None]
        self.sin, self.cos = ang.sin().bfloat16(), ang.cos().bfloat16()
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.cur = torch.zeros(batch, dtype=torch.long, device=dev)
        self.out = torch.zeros(new_tokens, batch, dtype=torch.int32, device=dev)
        self.mask_positions = torch.arange(self.S, device=dev)
        self.graph = None
        self.use_graph = cuda_graph
        self._ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def _all_reduce(self, x):
        if self.tp > 1:
            dist.all_reduce(x)
        return x

    def _embed(self, tok):
        if self.tp == 1:
            return self.wte[tok]
        local = tok - self.rank * self.vshard
        ok = (local >= 0) & (local < self.vshard)
        x = self.wte[local.clamp(0, self.vshard - 1)] * ok[..., None].to(self.wte.dtype)
        return self._all_reduce(x)

    def _select(self, h):
        hn = F.layer_norm(h, (self.cfg.hidden,), *self.ln_f, self.cfg.eps)
        logits = self.head(hn).float()
        if self.tp > 1:
            ids = torch.arange(self.vshard, device=self.dev) + self.rank * self.vshard
            logits = logits.masked_fill(ids >= self.cfg.vocab_size, -1e30)
        m, i = logits.max(dim=-1)
        if self.tp == 1:
            return i
        i = i + self.rank * self.vshard
        gm = m.clone()
        dist.all_reduce(gm, op=dist.ReduceOp.MAX)
        cand = torch.where(m >= gm, i, torch.full_like(i, 1 << 30))
        dist.all_reduce(cand, op=dist.ReduceOp.MIN)
        return cand

    def _block(self, x, L, prefill):
        cfg, H, D = self.cfg, self.H, self.D
        h = F.layer_norm(x, (cfg.hidden,), L["ln_w"], L["ln_b"], cfg.eps)
        qkv = L["qkv"](h)
        if prefill:
            B, S = self.B, self.P
            q, k, v = (t.reshape(B, S, H, D).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
            sin, cos = self.sin[:S], self.cos[:S]
            q, k = rotary(q, sin, cos, cfg.rotary_dim), rotary(k, sin, cos, cfg.rotary_dim)
            L["k"][:, :, :S] = k
            L["v"][:, :, :S] = v
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B * S, H * D)
        else:
            B = self.B
            q, k, v = (t.reshape(B, H, 1, D) for t in qkv.chunk(3, dim=-1))
            sin, cos = self.sin[self.pos], self.cos[self.pos]
            q, k = rotary(q, sin, cos, cfg.rotary_dim), rotary(k, sin, cos, cfg.rotary_dim)
            L["k"].index_copy_(2, self.pos, k)
            L["v"].index_copy_(2, self.pos, v)
            mask = (self.mask_positions <= self.pos)[None, None, None, :]
            a = F.scaled_dot_product_attention(q, L["k"], L["v"], attn_mask=mask).reshape(B, H * D)
        y = L["out"](a) + L["fc_out"](F.gelu(L["fc_in"](h)))
        return x + self._all_reduce(y) + L["fc_out_bias"]

    def _prefill(self, prompt):
        x = self._embed(prompt.reshape(-1).long())
        for L in self.layers:
            x = self._block(x, L, True)
        last = x.reshape(self.B, self.P, -1)[:, -1]
        tok = self._select(last)
        self.cur.copy_(tok)
        self.out[0].copy_(tok)

    def _decode_step(self):
        x = self._embed(self.cur)
        for L in self.layers:
            x = self._block(x, L, False)
        tok = self._select(x)
        self.pos.add_(1)
        self.cur.copy_(tok)
        self.out.index_copy_(0, self.pos - self.P, tok.to(torch.int32)[None])

    @torch.no_grad()
    def generate(self, prompt):
        prompt = prompt.to(self.dev, non_blocking=True)
        self.pos.fill_(self.P)
        self._ev[0].record()
        self._prefill(prompt)
        self._ev[1].record()
        if self.use_graph and self.graph is None:
            # capture one decode step (after a warm-up step on a side stream, as torch requires)
            saved = (self.pos.clone(), self.cur.clone(), self.out.clone())
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_step()
            torch.cuda.current_stream().wait_stream(s)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._decode_step()
            self.pos.copy_(saved[0]); self.cur.copy_(saved[1]); self.out.copy_(saved[2])
            self._ev[1].record()
        for _ in range(self.N - 1):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._decode_step()
        self._ev[2].record()
        res = self.out.t().contiguous().cpu().numpy()
        return res

    def prefill_ms(self):
        return self._ev[0].elapsed_time(self._ev[1])

    def decode_ms(self):
        return self._ev[1].elapsed_time(self._ev[2])
