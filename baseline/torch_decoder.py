"""Plain PyTorch (+cuBLAS, flash SDPA, NCCL) implementation of the benchmark configuration: the number this framework
has to match or beat on the same machine (the reference itself cannot run without Graphcore hardware).

Same model shape, same step: 16 micro-batches of 1 x 2048 tokens with gradient accumulation (optionally per-layer
activation checkpointing), bf16 parameters and compute with fp32 master weights and fp32 moments (fused AdamW on the
master copy, no per-micro-batch re-cast of the weights), Megatron-style tensor parallelism (column/row-parallel linears
with NCCL all-reduce, vocabulary-sharded embedding / head / cross-entropy), data parallelism as ONE all-reduce of a flat
gradient buffer per step, and the micro-batch (forward + backward) captured in a CUDA graph and replayed, as this
package's arm does. What a competent PyTorch user would run.  `python bench.py --impl torch` drives it.
"""
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


class _CopyToTP(torch.autograd.Function):  # forward identity, backward all-reduce
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):  # forward all-reduce, backward identity
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def rotary(x, sin, cos, rot):
    xr, xp = x[..., :rot], x[..., rot:]
    x1, x2 = xr[..., ::2], xr[..., 1::2]
    y = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)
    return torch.cat((y, xp), dim=-1)


class Block(nn.Module):
    def __init__(self, cfg, tp, group):
        super().__init__()
        self.cfg, self.tp, self.group = cfg, tp, group
        h, hd = cfg.hidden, cfg.heads // tp * cfg.head_dim
        self.ln = nn.LayerNorm(h, eps=cfg.eps)
        self.qkv = nn.Linear(h, 3 * hd, bias=False)
        self.out = nn.Linear(hd, h, bias=False)
        self.fc_in = nn.Linear(h, cfg.ffn // tp)
        self.fc_out = nn.Linear(cfg.ffn // tp, h, bias=False)
        self.fc_out_bias = nn.Parameter(torch.zeros(h))

    def forward(self, x, sin, cos):
        cfg = self.cfg
        B, S, _ = x.shape
        hloc = cfg.heads // self.tp
        h = self.ln(x)
        if self.tp > 1:
            h = _CopyToTP.apply(h, self.group)
        q, k, v = self.qkv(h).view(B, S, 3, hloc, cfg.head_dim).permute(2, 0, 3, 1, 4)
        q, k = rotary(q, sin, cos, cfg.rotary_dim), rotary(k, sin, cos, cfg.rotary_dim)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, -1)
        a = self.out(a)
        m = self.fc_out(F.gelu(self.fc_in(h)))
        y = a + m
        if self.tp > 1:
            y = _ReduceFromTP.apply(y, self.group)
        return x + y + self.fc_out_bias


class Model(nn.Module):
    def __init__(self, cfg, tp, group, tp_rank, recompute=True):
        super().__init__()
        self.cfg, self.tp, self.group, self.tp_rank = cfg, tp, group, tp_rank
        self.recompute = recompute
        self.vshard = -(-cfg.vocab_size // tp)
        self.wte = nn.Embedding(self.vshard, cfg.hidden)
        self.blocks = nn.ModuleList([Block(cfg, tp, group) for _ in range(cfg.layers)])
        self.ln_f = nn.LayerNorm(cfg.hidden, eps=cfg.eps)
        self.head = nn.Linear(cfg.hidden, self.vshard)
        inv = 1.0 / (10000 ** (torch.arange(0, cfg.rotary_dim, 2).float() / cfg.rotary_dim))
        ang = torch.outer(torch.arange(cfg.seq_len).float(), inv)
        self.register_buffer("sin", ang.sin()[None, None], persistent=False)
        self.register_buffer("cos", ang.cos()[None, None], persistent=False)

    def forward(self, tokens, labels):
        off = self.tp_rank * self.vshard
        idx = tokens - off
        ok = (idx >= 0) & (idx < self.vshard)
        x = self.wte(idx.clamp(0, self.vshard - 1)) * ok.unsqueeze(-1)
        if self.tp > 1:
            x = _ReduceFromTP.apply(x, self.group)
        for blk in self.blocks:
            x = checkpoint(blk, x, self.sin, self.cos, use_reentrant=False, preserve_rng_state=False) if self.recompute else blk(x, self.sin, self.cos)
        h = self.ln_f(x)
        if self.tp > 1:
            h = _CopyToTP.apply(h, self.group)
        logits = self.head(h).float().view(-1, self.vshard)  # loss in fp32
        if self.tp == 1:
            return F.cross_entropy(logits, labels.view(-1))
        # vocabulary-sharded cross entropy
        lab = labels.view(-1) - off
        inr = (lab >= 0) & (lab < self.vshard)
        mx = logits.max(dim=-1).values.detach()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
        z = logits - mx[:, None]
        se = _ReduceFromTP.apply(z.exp().sum(-1), self.group)
        picked = _ReduceFromTP.apply(z.gather(1, lab.clamp(0, self.vshard - 1)[:, None])[:, 0] * inr, self.group)
        return (se.log() - picked).mean()


class TorchTrainer:
    def __init__(self, cfg, micro_batches=16, lr=1e-4, recompute=True, cuda_graph=True):
        self.cfg, self.micro_batches = cfg, micro_batches
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        self.world, self.rank = world, rank
        tp, dp = cfg.tp, cfg.dp
        self.tp_group = self.dp_group = None
        if world > 1:
            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
            for g in range(dp):
                ranks = list(range(g * tp, (g + 1) * tp))
                grp = dist.new_group(ranks)
                if rank in ranks:
                    self.tp_group = grp
            for t in range(tp):
                ranks = list(range(t, world, tp))
                grp = dist.new_group(ranks)
                if rank in ranks:
                    self.dp_group = grp
        torch.manual_seed(1234 + rank % tp)
        dev = self.device = "cuda" if torch.cuda.is_available() else "cpu"  # the CPU path only smoke-tests the logic
        with torch.device(dev):
            self.model = Model(cfg, tp, self.tp_group, rank % tp, recompute=recompute).to(torch.bfloat16)
        params = sorted(self.model.parameters(), key=lambda p: p.dim() < 2)  # matrices (decayed) first, stable
        for p in params:
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.02)
        # bf16 parameters and gradients as views of two flat buffers (one collective per step, static addresses for the
        # captured graph); fp32 master copy for the optimizer
        total = sum(p.numel() for p in params)
        self.flat_w = torch.empty(total, dtype=torch.bfloat16, device=dev)
        self.flat_g = torch.zeros(total, dtype=torch.bfloat16, device=dev)
        off = 0
        for p in params:
            n = p.numel()
            self.flat_w[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_w[off:off + n].view_as(p)
            p.grad = self.flat_g[off:off + n].view_as(p)
            off += n
        n_decay = sum(p.numel() for p in params if p.dim() >= 2)
        self.master = self.flat_w.float()
        self.master_grad = torch.zeros_like(self.master)
        groups = []
        for lo, hi, wd in ((0, n_decay, 0.01), (n_decay, total, 0.0)):
            parts = []
            for a in range(lo, hi, 1 << 30):  # pieces below 2^31 elements
                b = min(a + (1 << 30), hi)
                part = self.master[a:b]
                part.grad = self.master_grad[a:b]
                parts.append(part)
            if parts:
                groups.append({"params": parts, "weight_decay": wd})
        self.opt = torch.optim.AdamW(groups, lr=lr, betas=(0.9, 0.95), eps=1e-5, fused=dev == "cuda")
        self.tokens_per_step = micro_batches * cfg.seq_len * dp
        self.cuda_graph = bool(cuda_graph) and dev == "cuda"
        self.graph = None
        self.graph_note = "off"
        self._static_tokens = torch.zeros(1, cfg.seq_len + 1, dtype=torch.long, device=dev)
        self._static_loss = None
        self._eager_steps = 0

    def _micro_batch(self, t):
        loss = self.model(t[:, :-1], t[:, 1:])
        (loss / self.micro_batches).backward()  # accumulates into the flat bf16 gradient buffer
        return loss.detach()

    def _try_capture(self):
        """Capture one micro-batch (forward + backward, collectives included) after a warm-up on a side stream."""
        try:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                self._static_loss = self._micro_batch(self._static_tokens)
            self.graph, self.graph_note = g, "micro-batch replayed from a CUDA graph"
        except Exception as e:  # capture is not always possible (an op that synchronises): stay eager and say so
            self.graph, self.graph_note = None, f"eager ({type(e).__name__} during capture)"
            self.cuda_graph = False
            torch.cuda.synchronize()
        self.flat_g.zero_()

    def step_device(self, tokens):
        """tokens: (micro_batches, 1, 1, seq+1) int32 on the device. Returns per-micro-batch losses (device)."""
        if self.cuda_graph and self.graph is None and self._eager_steps >= 1:
            self._try_capture()
        losses = []
        for i in range(self.micro_batches):
            t = tokens[i].reshape(1, -1).long()
            if self.graph is not None:
                self._static_tokens.copy_(t)
                self.graph.replay()
                losses.append(self._static_loss.clone())
            else:
                losses.append(self._micro_batch(t))
        self._eager_steps += 1
        if self.cfg.dp > 1:
            dist.all_reduce(self.flat_g, op=dist.ReduceOp.AVG, group=self.dp_group)  # one flat bucket
        self.master_grad.copy_(self.flat_g)
        self.flat_g.zero_()
        self.opt.step()
        self.flat_w.copy_(self.master)
        return torch.stack(losses)

    def step(self, host_tokens):
        return float(self.step_device(host_tokens.to(self.device, non_blocking=True)).float().mean().item())
