"""Plain PyTorch pipeline-parallel x data-parallel training step: the bar for `bench.py --mode pipeline`.

Llama-shape decoder (RMSNorm, rotary attention, SwiGLU) split into equal runs of layers, one process per stage and data-
parallel replica (`rank = replica * stages + stage`, the layout of this package's `PipelineTrainer`). Non-interleaved 1F1B
schedule over `micro_batches` micro-batches of one sequence: a stage runs `stages - stage - 1` forward passes ahead, then
alternates one forward with one backward, then drains; activations and their gradients cross stage boundaries with
`torch.distributed` send / recv (NCCL p2p). bf16 parameters and gradients in flat buffers, fp32 master weights with fused
AdamW, one flat gradient all-reduce over the data-parallel group per step. cuBLAS GEMMs, flash SDPA attention.
"""
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _rope(x, sin, cos):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        h, hd = cfg.hidden, cfg.heads * cfg.head_dim
        self.cfg = cfg
        self.n1 = nn.RMSNorm(h, eps=cfg.eps)
        self.qkv = nn.Linear(h, 3 * hd, bias=False)
        self.out = nn.Linear(hd, h, bias=False)
        self.n2 = nn.RMSNorm(h, eps=cfg.eps)
        self.gate = nn.Linear(h, cfg.ffn, bias=False)
        self.up = nn.Linear(h, cfg.ffn, bias=False)
        self.down = nn.Linear(cfg.ffn, h, bias=False)

    def forward(self, x, sin, cos):
        cfg = self.cfg
        B, S, _ = x.shape
        q, k, v = self.qkv(self.n1(x)).view(B, S, 3, cfg.heads, cfg.head_dim).permute(2, 0, 3, 1, 4)
        q, k = _rope(q, sin, cos), _rope(k, sin, cos)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, -1)
        x = x + self.out(a)
        h = self.n2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class Stage(nn.Module):
    def __init__(self, cfg, stage, stages):
        super().__init__()
        self.cfg, self.first, self.last = cfg, stage == 0, stage == stages - 1
        per = cfg.layers // stages
        if self.first:
            self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(per)])
        if self.last:
            self.norm = nn.RMSNorm(cfg.hidden, eps=cfg.eps)
            self.head = nn.Linear(cfg.hidden, cfg.vocab_size, bias=False)
        inv = 1.0 / (10000 ** (torch.arange(0, cfg.head_dim, 2).float() / cfg.head_dim))
        ang = torch.outer(torch.arange(cfg.seq_len).float(), inv)
        self.register_buffer("sin", ang.sin()[None, None], persistent=False)
        self.register_buffer("cos", ang.cos()[None, None], persistent=False)

    def forward(self, x, labels=None):
        if self.first:
            x = self.wte(x)
        for blk in self.blocks:
            x = blk(x, self.sin, self.cos)
        if self.last:
            logits = self.head(self.norm(x)).float().view(-1, self.cfg.vocab_size)
            return F.cross_entropy(logits, labels.view(-1))
        return x


class TorchPipelineTrainer:
    def __init__(self, cfg, stages, micro_batches=32, lr=1e-4):
        self.cfg, self.stages, self.micro_batches = cfg, stages, micro_batches
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        self.rank, self.world = rank, world
        self.stage, self.replica = rank % stages, rank // stages
        self.dp = world // stages
        self.dp_group = None
        for s in range(stages):
            grp = dist.new_group(list(range(s, world, stages)))
            if s == self.stage:
                self.dp_group = grp
        torch.manual_seed(4321 + self.stage)
        with torch.device("cuda"):
            self.model = Stage(cfg, self.stage, stages).to(torch.bfloat16)
        params = list(self.model.parameters())
        for p in params:
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.02)
        total = sum(p.numel() for p in params)
        self.flat_w = torch.empty(total, dtype=torch.bfloat16, device="cuda")
        self.flat_g = torch.zeros(total, dtype=torch.bfloat16, device="cuda")
        off = 0
        for p in params:
            n = p.numel()
            self.flat_w[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_w[off:off + n].view_as(p)
            p.grad = self.flat_g[off:off + n].view_as(p)
            off += n
        self.master = self.flat_w.float()
        self.master_grad = torch.zeros_like(self.master)
        parts = []
        for a in range(0, total, 1 << 30):
            part = self.master[a:min(a + (1 << 30), total)]
            part.grad = self.master_grad[a:min(a + (1 << 30), total)]
            parts.append(part)
        self.opt = torch.optim.AdamW(parts, lr=lr, betas=(0.9, 0.95), eps=1e-5, weight_decay=0.01, fused=True)
        self.tokens_per_step = micro_batches * cfg.seq_len * self.dp
        self.act_shape = (1, cfg.seq_len, cfg.hidden)

    def _peer(self, stage):
        return self.replica * self.stages + stage

    # -- stage-boundary exchanges: a send and a receive that face each other on two ranks go out as one batch --------------
    def _exchange(self, send=None, send_to=None, recv_from=None):
        ops, buf = [], None
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), self._peer(send_to)))
        if recv_from is not None:
            buf = torch.empty(self.act_shape, dtype=torch.bfloat16, device="cuda")
            ops.append(dist.P2POp(dist.irecv, buf, self._peer(recv_from)))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return buf

    def step_device(self, tokens):
        """tokens: (micro_batches, 1, 1, seq + 1) int32 on the device (read by the first and the last stage).
        Non-interleaved 1F1B: warm-up forwards, steady one-forward-one-backward, cool-down backwards."""
        S, s, M = self.stages, self.stage, self.micro_batches
        first, last = s == 0, s == S - 1
        pending, losses = [], []
        state = {"f": 0}

        def forward(x_in):
            t = tokens[state["f"]].reshape(1, -1).long()
            state["f"] += 1
            if first:
                out = self.model(t[:, :-1], t[:, 1:] if last else None)
            else:
                x_in.requires_grad_(True)
                out = self.model(x_in, t[:, 1:] if last else None)
            if last:
                losses.append(out.detach())
            pending.append((x_in, out))
            return out

        def backward(grad_out):
            x_in, out = pending.pop(0)
            if last:
                (out / M).backward()
            else:
                out.backward(grad_out)
            return None if first else x_in.grad

        warm = min(S - s - 1, M)
        remaining = M - warm
        for _ in range(warm):
            x_in = None if first else self._exchange(recv_from=s - 1)
            out = forward(x_in)
            if not last:
                self._exchange(send=out.detach(), send_to=s + 1)
        x_in = None
        if remaining > 0 and not first:
            x_in = self._exchange(recv_from=s - 1)
        for i in range(remaining):
            out = forward(x_in)
            grad_out = None if last else self._exchange(send=out.detach(), send_to=s + 1, recv_from=s + 1)
            grad_in = backward(grad_out)
            if first:
                x_in = None
            elif i == remaining - 1:
                self._exchange(send=grad_in, send_to=s - 1)
            else:
                x_in = self._exchange(send=grad_in, send_to=s - 1, recv_from=s - 1)
        for _ in range(warm):
            grad_out = None if last else self._exchange(recv_from=s + 1)
            grad_in = backward(grad_out)
            if not first:
                self._exchange(send=grad_in, send_to=s - 1)
        if self.dp > 1:
            dist.all_reduce(self.flat_g, op=dist.ReduceOp.AVG, group=self.dp_group)
        self.master_grad.copy_(self.flat_g)
        self.flat_g.zero_()
        self.opt.step()
        self.flat_w.copy_(self.master)
        return torch.stack(losses) if losses else None

    def step(self, host_tokens):
        out = self.step_device(host_tokens.cuda(non_blocking=True))
        return float(out.float().mean().item()) if out is not None else None
