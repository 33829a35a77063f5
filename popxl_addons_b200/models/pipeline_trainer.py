"""Pipeline-parallel training of the decoder family: the layers are split evenly over `stages` device slots, every
replica spans `stages` processes (one per GPU), replicas are data-parallel.

    with pipelined_execution(micro_batches) as p:
        stage 0      (slot 0)      tokens -> embedding -> first layers -> copy to slot 1
        stage s      (slot s)      layers of slot s -> copy to slot s+1
        stage S-1    (slot S-1)    last layers -> head -> fused cross-entropy -> head backward -> backward of the last
                                   layers (activations still at hand) -> copy of the gradient to slot S-2
        stage S-1+k  (slot S-1-k)  backward of the layers of that slot from stashed activations -> copy / embedding
                                   backward
    optimizer: every slot updates its own parameters (gradient mean over the data-parallel group, AdamW on fp32 master
    weights; sharded over the group and fused into one kernel per parameter where possible)

In steady state all slots work at once on different micro-batches; stage boundaries are batched NCCL send/recv.
Weight gradients accumulate as running means inside the gradient graphs, per-layer recomputation keeps the stash to
one activation per layer and micro-batch in flight. Without a launcher the same program runs in one process with all
slots in it (CPU oracle).

Parity: the reference composes the same program from popxl_addons/transforms/pipelining.py:26-508 (stages, stash and
restore) with its autodiff / recomputation transforms; its device slots are the IPUs of one replica.
"""
import os
from typing import List, Optional

import numpy as np
import torch

from .. import xl
from ..named_tensors import NamedTensors
from ..patterns import apply_pre_alias_patterns
from ..streams import InputStreams, OutputStreams
from ..task_session import TaskSession
from ..transforms.autodiff import autodiff_with_accumulation
from ..transforms.pipelining import pipelined_execution
from ..transforms.recomputation import recompute_graph
from ..xl import ops
from .decoder import DecoderBlock, DecoderConfig, DecoderEmbedding, DecoderHead, _Parallel, rotary_tables
from .trainer import build_optimizer

__all__ = ["PipelineTrainer"]


class PipelineTrainer:
    def __init__(self, cfg: DecoderConfig, stages: int = 4, micro_batches: int = 32, micro_batch_size: int = 1,
                 device: str = "auto", seed: int = 0, lr: float = 1e-4, weight_decay: float = 0.01, beta1: float = 0.9,
                 beta2: float = 0.95, eps: float = 1e-5, recompute: bool = True,
                 optimizer_state_dtype: xl.dtype = xl.float32, shard_optimizer: bool = True,
                 fused_collectives: bool = True, use_native: Optional[bool] = None,
                 prune_recompute: Optional[bool] = None):
        if cfg.tp != 1:
            raise ValueError("PipelineTrainer combines pipeline and data parallelism (tp must be 1)")
        if cfg.layers % stages:
            raise ValueError(f"{cfg.layers} layers cannot be split evenly over {stages} stages")
        n_pipeline_stages = 2 * stages - 1
        if micro_batches < 2 * n_pipeline_stages:
            raise ValueError(f"{stages} device slots make {n_pipeline_stages} pipeline stages: at least "
                             f"{2 * n_pipeline_stages} micro-batches per step are needed")
        self.cfg, self.stages = cfg, stages
        self.micro_batches, self.micro_batch_size = micro_batches, micro_batch_size
        world = int(os.environ.get("WORLD_SIZE", "1"))
        distributed = world > 1
        if distributed and world != stages * cfg.dp:
            raise ValueError(f"WORLD_SIZE={world} must equal stages*dp={stages * cfg.dp}")
        np.random.seed(seed)
        self.ir = (xl.Ir(replication="popdist", devices_per_replica=stages) if distributed
                   else xl.Ir(replication=cfg.dp))
        self.hp = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)
        self.recompute = recompute
        # the recomputed forward pass leaves out what only leads to the block's output (XL_PRUNE_RECOMPUTE=1)
        self.prune_recompute = (os.environ.get("XL_PRUNE_RECOMPUTE", "0") == "1") if prune_recompute is None \
            else bool(prune_recompute)
        self.state_dtype = optimizer_state_dtype
        self.shard_optimizer = shard_optimizer and cfg.dp > 1
        self.fused_collectives = fused_collectives
        self._build()
        apply_pre_alias_patterns(self.ir)
        self.session = TaskSession(self.inputs, self.outputs, self.state, 1, self.ir, device, use_native=use_native)
        self.tokens_per_step = micro_batches * micro_batch_size * cfg.seq_len * cfg.dp
        slot = self.session.slot
        self.has_loss = slot is None or slot == stages - 1

    def _build(self):
        cfg, ir, S = self.cfg, self.ir, self.stages
        T = self.micro_batch_size * cfg.seq_len
        dt, f32 = cfg.xl_dtype, xl.float32
        per = cfg.layers // S
        slot_of_layer = [i // per for i in range(cfg.layers)]
        with ir.main_graph:
            par = _Parallel(cfg)
            tok_shape = ((self.micro_batch_size, cfg.seq_len + 1), xl.int32)
            self.inputs = InputStreams(tokens=tok_shape, labels=tok_shape)
            self.outputs = OutputStreams(loss=((), xl.float32))
            sin, cos = rotary_tables(cfg)
            x_spec = xl.TensorSpec((T, cfg.hidden), dt)
            tok_spec = xl.TensorSpec((T,), xl.int32)
            emb_facts, emb_graph = DecoderEmbedding(cfg).create_graph(tok_spec)
            blk_facts, blk_graph = DecoderBlock(cfg).create_graph(x_spec, sin.spec, cos.spec)
            head_facts, head_graph = DecoderHead(cfg).create_graph(x_spec)
            emb_dfacts, emb_grad = autodiff_with_accumulation(emb_graph, emb_graph.args.tensors, accum_dtype=f32)
            blk_dfacts, blk_grad = autodiff_with_accumulation(blk_graph, blk_graph.args.tensors,
                                                              grads_required=[blk_graph.graph.inputs[0]],
                                                              accum_dtype=f32)
            if self.recompute:
                blk_grad = recompute_graph(blk_grad, prune_forward=self.prune_recompute)
            head_dfacts, head_grad = autodiff_with_accumulation(head_graph, head_graph.args.tensors,
                                                                grads_required=[head_graph.graph.inputs[0]],
                                                                accum_dtype=f32)
            # variables live on the slot that uses them
            with xl.ipu(0):
                emb_vars = emb_facts.init("embedding")
            with xl.ipu(S - 1):
                head_vars = head_facts.init("head")
            blk_vars = []
            for i in range(cfg.layers):
                with xl.ipu(slot_of_layer[i]):
                    blk_vars.append(blk_facts.init(f"layer{i}"))
            with xl.ipu(0):
                emb_acc = emb_dfacts.init("embedding.grad")
            with xl.ipu(S - 1):
                head_acc = head_dfacts.init("head.grad")
            blk_acc = []
            for i in range(cfg.layers):
                with xl.ipu(slot_of_layer[i]):
                    blk_acc.append(blk_dfacts.init(f"layer{i}.grad"))

            calls: List = [None] * cfg.layers

            def forward_layers(x, slot):
                for i in range(slot * per, (slot + 1) * per):
                    calls[i] = blk_graph.bind(blk_vars[i]).call_with_info(x, sin, cos)
                    x = calls[i].outputs[0]
                return x

            with pipelined_execution(self.micro_batches) as p:
                with p.stage(0), xl.ipu(0):
                    tok = ops.host_load(self.inputs.tokens)
                    inp = ops.reshape(tok[:, :-1], (T,))
                    emb_call = emb_graph.bind(emb_vars).call_with_info(inp)
                    x = forward_layers(emb_call.outputs[0], 0)
                    if S > 1:
                        x = x.copy_to_ipu(1)
                for s in range(1, S - 1):
                    with p.stage(s), xl.ipu(s):
                        x = forward_layers(x, s).copy_to_ipu(s + 1)
                with p.stage(S - 1), xl.ipu(S - 1):
                    if S > 1:
                        x = forward_layers(x, S - 1)
                        lab_src = ops.host_load(self.inputs.labels)
                    else:
                        lab_src = tok
                    lab = ops.reshape(lab_src[:, 1:], (T,))
                    head_call = head_graph.bind(head_vars).call_with_info(x)
                    loss, dlogits = ops.cross_entropy_with_grad(head_call.outputs[0], lab, 1.0)
                    ops.host_store(self.outputs.loss, ops.cast(loss, xl.float32))
                    (dx,) = head_grad.bind(head_acc).call(dlogits, args=head_grad.grad_graph_info.inputs_dict(head_call))
                    for i in reversed(range((S - 1) * per, S * per)):
                        (dx,) = blk_grad.bind(blk_acc[i]).call(dx, args=blk_grad.grad_graph_info.inputs_dict(calls[i]))
                    if S > 1:
                        dx = dx.copy_to_ipu(S - 2)
                    else:
                        emb_grad.bind(emb_acc).call(dx, args=emb_grad.grad_graph_info.inputs_dict(emb_call))
                for k in range(1, S):
                    slot = S - 1 - k
                    with p.stage(S - 1 + k), xl.ipu(slot):
                        for i in reversed(range(slot * per, (slot + 1) * per)):
                            (dx,) = blk_grad.bind(blk_acc[i]).call(
                                dx, args=p.stash_and_restore_activations(calls[i], blk_grad.grad_graph_info))
                        if slot > 0:
                            dx = dx.copy_to_ipu(slot - 1)
                        else:
                            emb_grad.bind(emb_acc).call(
                                dx, args=p.stash_and_restore_activations(emb_call, emb_grad.grad_graph_info))

            groups = ([("embedding", emb_vars, emb_acc), ("head", head_vars, head_acc)] +
                      [(f"layer{i}", blk_vars[i], blk_acc[i]) for i in range(cfg.layers)])

            def slot_of(name: str) -> int:
                if name == "embedding":
                    return 0
                if name == "head":
                    return S - 1
                return slot_of_layer[int(name[len("layer"):])]

            self.master, opt_state = build_optimizer(ir, cfg, par, groups, self.hp, self.state_dtype,
                                                     self.shard_optimizer, self.fused_collectives, slot_of=slot_of)
            for name, _, atree in groups:
                with xl.ipu(slot_of(name)):
                    ops.var_updates.accumulator_zero_(atree.mean_accum_counter)

        weights = NamedTensors(embedding=emb_vars, head=head_vars)
        for i in range(cfg.layers):
            weights.insert(f"layer{i}", blk_vars[i])
        state = NamedTensors(model=weights)
        state.insert("master", NamedTensors.from_dict({k.replace(".", "_"): v for k, v in self.master.items()}))
        state.insert("adam", NamedTensors.from_dict({k.replace(".", "_"): v for k, v in opt_state.items()}))
        self.state, self.weights = state, weights
        self.ir.num_host_transfers = self.micro_batches

    # ------------------------------------------------------------------------------------------------------------
    def step(self, tokens) -> Optional[float]:
        """One optimizer step. `tokens`: int32 `(micro_batches, [replicas,] micro_batch_size, seq_len + 1)` on the
        host. Returns the mean loss of this replica's micro-batches on the processes that compute it (the last
        slot; every process in the single-process simulation), None elsewhere."""
        out = self.session.run({self.inputs.tokens: tokens, self.inputs.labels: tokens})
        if not self.has_loss:
            return None
        return float(np.mean(out[self.outputs.loss]))

    def step_device(self, tokens_on_device: torch.Tensor):
        out = self.session.run({self.inputs.tokens: tokens_on_device, self.inputs.labels: tokens_on_device}, fetch=False)
        return out.get(self.outputs.loss)

    def synthetic_tokens(self, seed: int = 0, pinned: bool = True) -> torch.Tensor:
        """Uniform random token ids of the step's shape for this process (all slots of a replica see the same data)."""
        replica = int(os.environ.get("RANK", "0")) // self.stages if self.session.distributed else 0
        g = torch.Generator().manual_seed(seed + replica)
        local = 1 if self.session.distributed else self.cfg.dp
        shape = (self.micro_batches, local, self.micro_batch_size, self.cfg.seq_len + 1)
        t = torch.randint(0, self.cfg.vocab_size, shape, generator=g, dtype=torch.int32)
        if pinned and torch.cuda.is_available():
            t = t.pin_memory()
        return t
