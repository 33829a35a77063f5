"""Training program for the decoder family, composed from the add-on pieces the way a reference user would:

    facts, fwd   = Block().create_graph(x_spec, sin, cos)            # one graph, shared by all layers
    dfacts, grad = autodiff_with_accumulation(fwd, fwd.args.tensors, grads_required=[x])   (+ recompute_graph)
    micro-batch graph (repeated `micro_batches` times per step):
        host_load tokens -> embedding -> L x block forward -> head -> fused cross-entropy (loss + dlogits)
        -> head backward -> L x block backward (recomputing the block) -> embedding backward;
        weight gradients are folded into running-mean accumulators inside the gradient graphs
    after the loop: per parameter, reduce over the data-parallel group (reduce-scatter when the optimizer state is
    sharded: replicated tensor sharding), AdamW on fp32 master weights, all-gather of the updated 16-bit weights.

Layout: one process per GPU (`torchrun`), replica = rank, TP ranks consecutive. On a single process without a launcher
the same program runs all replicas in-process (CPU oracle / tests).
"""
import os
import time
from typing import Dict, Optional

import numpy as np
import torch

from .. import xl
from ..named_tensors import NamedTensors
from ..ops.cross_entropy_sharded_loss import cross_entropy_sharded_with_grad
from ..optimizers.adam import AdamOptimizerStep
from ..patterns import apply_pre_alias_patterns
from ..rts import reduce_replica_sharded_tensor
from ..task_session import TaskSession
from ..transforms.autodiff import autodiff_with_accumulation
from ..transforms.recomputation import recompute_graph
from ..streams import InputStreams, OutputStreams
from ..layers.embedding import model_vocab_offsets
from ..xl import ops
from .decoder import DecoderBlock, DecoderConfig, DecoderEmbedding, DecoderHead, _Parallel, rotary_tables

__all__ = ["DecoderTrainer"]


def build_optimizer(ir, cfg, par, groups, hp, state_dtype, shard_optimizer, fused_collectives, slot_of=None,
                    reduce_replicated_over=None):
    """Emit the AdamW update of every parameter of `groups` (`(name, weights, accumulators)` triples) into the
    current graph: fp32 master weights and moments, sharded over the data-parallel group when `shard_optimizer`
    (as one fused reduce-scatter + AdamW + all-gather kernel per parameter when `fused_collectives`), otherwise a
    gradient all-reduce followed by a replicated update. `slot_of(name)` places a group's update on a device slot
    (pipeline parallel). `reduce_replicated_over`: replica grouping over which the gradients of parameters that are
    replicated across it are only partial sums and have to be added up first (the TP group under sequence
    parallelism, where norm weights and output biases see tokens/tp rows per rank).
    Returns `(master weights by name, optimizer state by name)`."""
    import contextlib

    def placed(name):
        return xl.ipu(slot_of(name)) if slot_of is not None else contextlib.nullcontext()

    masters: Dict[str, xl.Variable] = {}
    opt_state = {}
    opt_graphs: Dict[tuple, tuple] = {}

    fused_jobs = []  # (weight, accumulator, master shard, decay, name): emitted together below
    for group_name, wtree, atree in groups:
        wd, ad = wtree.to_dict(), atree.accum.to_dict()
        with placed(group_name):
            for pname, w in wd.items():
                g = ad[pname]
                full = f"{group_name}.{pname}"
                if reduce_replicated_over is not None and (w.replica_grouping is None
                                                           or w.replica_grouping.num_groups == 1):
                    g = ops.collectives.replicated_all_reduce_(g, "add", reduce_replicated_over)
                decay = hp["weight_decay"] if w.rank >= 2 else 0.0
                host = ir.initial_values[w]
                if isinstance(host, xl.LazyInit):
                    host32 = host.astype(np.float32)  # same recipe and seed, drawn in fp32
                else:
                    host32 = (host.float() if isinstance(host, torch.Tensor)
                              else torch.tensor(np.asarray(host)).float()).numpy()
                rg = w.replica_grouping
                shardable = shard_optimizer and w.nelms % cfg.dp == 0
                fusable = (shardable and fused_collectives and w.dtype in (xl.bfloat16, xl.float16)
                           and (w.nelms // cfg.dp) % 4 == 0)
                if fusable:
                    master, _ = xl.replica_sharded_variable(host32, xl.float32, f"master.{full}",
                                                            replica_grouping=rg, shard_grouping=par.dp_group)
                    masters[full] = master
                    w.symmetric_group = par.dp_group
                    g.symmetric_group = par.dp_group
                    fused_jobs.append((w, g, master, decay, full, rg, group_name))
                    continue
                if shardable:
                    g = reduce_replica_sharded_tensor(g, "mean", par.dp_group, par.dp_group)
                    master, _ = xl.replica_sharded_variable(host32, xl.float32, f"master.{full}",
                                                            replica_grouping=rg, shard_grouping=par.dp_group)
                    key = ("sharded", master.shape, decay)
                else:
                    if cfg.dp > 1:
                        g = ops.collectives.replicated_all_reduce(g, "mean", par.dp_group)
                    master = xl.variable(host32, xl.float32, f"master.{full}", replica_grouping=rg)
                    key = ("full", tuple(w.shape), decay)
                masters[full] = master
                if key not in opt_graphs:
                    with xl.ipu(None):  # the graph is shared by parameters on different slots
                        ofacts, ograph = AdamOptimizerStep().create_graph(
                            master, g, rg, lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"], eps=hp["eps"],
                            weight_decay=decay, first_order_dtype=state_dtype, bias_correction=True)
                    opt_graphs[key] = (ofacts, ograph)
                ofacts, ograph = opt_graphs[key]
                ostate = ofacts.init(f"adam.{full}")
                ograph.bind(ostate).call(master, g)
                opt_state[full] = ostate
                new_w = ops.cast(master, w.dtype)
                if shardable:
                    new_w = ops.collectives.replicated_all_gather(new_w, par.dp_group, output_shape=w.shape)
                ops.var_updates.copy_var_update_(w, new_w)
    # one fused kernel per bucket (= per group: a layer, the embedding, the head): reduce-scatter + AdamW + all-gather of
    # all its parameters; only the first call of a device slot waits for all replicas' accumulators and only the last one
    # for all replicas' weight shards
    from ..optimizers.rts_adam import RTSAdamBucketStep

    buckets: Dict[str, list] = {}
    for job in fused_jobs:
        buckets.setdefault(job[6], []).append(job)
    order = list(buckets)
    for j, group_name in enumerate(order):
        jobs = buckets[group_name]
        same = [k for k, gname in enumerate(order) if slot_of is None or slot_of(gname) == slot_of(group_name)]
        first, last = j == same[0], j == same[-1]
        ws, gs, ms_ = [job[0] for job in jobs], [job[1] for job in jobs], [job[2] for job in jobs]
        decays = tuple(job[3] for job in jobs)
        names = [job[4][len(group_name) + 1:] for job in jobs]
        rgs = [job[5] for job in jobs]
        key = ("bucket", tuple(tuple(w.shape) for w in ws), decays, tuple(names), first, last)
        if key not in opt_graphs:
            with xl.ipu(None):
                opt_graphs[key] = RTSAdamBucketStep().create_graph(
                    ws, gs, ms_, names, par.dp_group, rgs, lr=hp["lr"], weight_decays=decays, beta1=hp["beta1"],
                    beta2=hp["beta2"], eps=hp["eps"], first_order_dtype=state_dtype, sync_before=first, sync_after=last)
        ofacts, ograph = opt_graphs[key]
        with placed(group_name):
            ostate = ofacts.init(f"adam.{group_name}")
            ograph.bind(ostate).call(*ws, *gs, *ms_)
        opt_state[group_name] = ostate
    return masters, opt_state


class DecoderTrainer:
    def __init__(self, cfg: DecoderConfig, micro_batches: int = 16, micro_batch_size: int = 1, device: str = "auto",
                 seed: int = 0, lr: float = 1e-4, weight_decay: float = 0.01, beta1: float = 0.9, beta2: float = 0.95,
                 eps: float = 1e-5, recompute: bool = True, optimizer_state_dtype: xl.dtype = xl.float32,
                 shard_optimizer: bool = True, use_native: Optional[bool] = None, fused_collectives: bool = True, cuda_graphs: bool = True,
                 prune_recompute: Optional[bool] = None):
        self.cfg = cfg
        self.micro_batches = micro_batches
        self.micro_batch_size = micro_batch_size
        world = int(os.environ.get("WORLD_SIZE", "1"))
        distributed = world > 1
        if distributed and world != cfg.tp * cfg.dp:
            raise ValueError(f"WORLD_SIZE={world} must equal tp*dp={cfg.tp * cfg.dp}")
        np.random.seed(seed)
        self.ir = xl.Ir(replication="popdist" if distributed else cfg.tp * cfg.dp)
        self.hp = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)
        self.recompute = recompute
        # the recomputed forward pass leaves out what only leads to the block's output (XL_PRUNE_RECOMPUTE=1)
        self.prune_recompute = (os.environ.get("XL_PRUNE_RECOMPUTE", "0") == "1") if prune_recompute is None \
            else bool(prune_recompute)
        self.state_dtype = optimizer_state_dtype
        self.shard_optimizer = shard_optimizer and cfg.dp > 1
        self.fused_collectives = fused_collectives
        self.cuda_graphs = cuda_graphs
        t0 = time.perf_counter()
        self._build()
        apply_pre_alias_patterns(self.ir)
        self.fused_gemm_collectives = 0
        # GEMM + all-reduce as one kernel (the pulling form: partial tiles stay local, NVSwitch adds them on the way into
        # the rank that owns the rows) up to this TP width; XL_FUSE_GEMM_AR=0 keeps GEMM and NCCL all-reduce separate
        fuse_up_to = int(os.environ.get("XL_FUSE_GEMM_AR_MAX_TP", "8"))
        if (fused_collectives and 1 < cfg.tp <= fuse_up_to and os.environ.get("XL_FUSE_GEMM_AR", "1") != "0"):
            from ..parallel import fuse_gemm_collectives

            self.fused_gemm_collectives = fuse_gemm_collectives(self.ir)
        self.fused_sequence_parallel = 0
        if fused_collectives and cfg.sp and os.environ.get("XL_FUSE_SP", "1") != "0":
            from ..parallel import fuse_sequence_parallel_collectives

            self.fused_sequence_parallel = fuse_sequence_parallel_collectives(self.ir)
        from ..parallel import fuse_matmul_sums

        self.fused_matmul_sums = fuse_matmul_sums(self.ir)  # what the collective fusion left: c = a1 @ w1 + a2 @ w2
        # XL_ASYNC_COLLECTIVES=1: all-reduces run asynchronously, and each graph is reordered so that the ops that do not
        # need an all-reduce's result (the weight-gradient GEMMs of a block) are issued before the ops that do
        self.async_collectives = cfg.tp > 1 and os.environ.get("XL_ASYNC_COLLECTIVES", "0") == "1"
        self.overlap_moves = 0
        if self.async_collectives:
            from ..parallel import schedule_collective_overlap

            self.overlap_moves = schedule_collective_overlap(self.ir)
        self.build_seconds = time.perf_counter() - t0
        self.session = TaskSession(self.inputs, self.outputs, self.state, 1, self.ir, device, use_native=use_native)
        if self.async_collectives and hasattr(self.session.comm, "async_collectives"):
            self.session.comm.async_collectives = True
        self.tokens_per_step = micro_batches * micro_batch_size * cfg.seq_len * cfg.dp

    # ------------------------------------------------------------------------------------------------------------
    def _build(self):
        cfg, ir = self.cfg, self.ir
        T = self.micro_batch_size * cfg.seq_len
        dt = cfg.xl_dtype
        with ir.main_graph:
            par = _Parallel(cfg)
            self.inputs = InputStreams(tokens=((self.micro_batch_size, cfg.seq_len + 1), xl.int32))
            self.outputs = OutputStreams(loss=((), xl.float32))
            sin, cos = rotary_tables(cfg)
            x_spec = xl.TensorSpec((T // cfg.tp if cfg.sp else T, cfg.hidden), dt)  # rows of the residual stream
            tok_spec = xl.TensorSpec((T,), xl.int32)

            # ---- graphs (one per distinct computation, shared by all layers) -----------------------------------
            emb_facts, emb_graph = DecoderEmbedding(cfg).create_graph(
                tok_spec, *( [xl.TensorSpec((), xl.int32)] if cfg.tp > 1 else []))
            blk_facts, blk_graph = DecoderBlock(cfg).create_graph(x_spec, sin.spec, cos.spec)
            head_facts, head_graph = DecoderHead(cfg).create_graph(x_spec)
            f32 = xl.float32
            emb_dfacts, emb_grad = autodiff_with_accumulation(emb_graph, emb_graph.args.tensors, accum_dtype=f32)
            blk_dfacts, blk_grad = autodiff_with_accumulation(blk_graph, blk_graph.args.tensors,
                                                              grads_required=[blk_graph.graph.inputs[0]],
                                                              accum_dtype=f32)
            if self.recompute:
                blk_grad = recompute_graph(blk_grad, prune_forward=self.prune_recompute)
            head_dfacts, head_grad = autodiff_with_accumulation(head_graph, head_graph.args.tensors,
                                                                grads_required=[head_graph.graph.inputs[0]],
                                                                accum_dtype=f32)

            # ---- variables -------------------------------------------------------------------------------------
            emb_vars, head_vars = emb_facts.init("embedding"), head_facts.init("head")
            blk_vars = [blk_facts.init(f"layer{i}") for i in range(cfg.layers)]
            emb_acc, head_acc = emb_dfacts.init("embedding.grad"), head_dfacts.init("head.grad")
            blk_acc = [blk_dfacts.init(f"layer{i}.grad") for i in range(cfg.layers)]
            offset_var = None
            if cfg.tp > 1:
                offs = model_vocab_offsets(cfg.vocab_size, cfg.tp).astype(np.int32)
                offset_var = xl.variable(offs, xl.int32, "vocab_offset", replica_grouping=par.dp_group)

            # ---- micro-batch graph -----------------------------------------------------------------------------
            weights = NamedTensors(embedding=emb_vars, head=head_vars)
            accums = NamedTensors(embedding=emb_acc, head=head_acc)
            for i in range(cfg.layers):
                weights.insert(f"layer{i}", blk_vars[i])
                accums.insert(f"layer{i}", blk_acc[i])
            mb = ir.create_empty_graph("micro_batch")
            flat_w, flat_a = weights.to_dict(), accums.to_dict()
            with mb:
                w_in = {k: xl.graph_input(v.shape, v.dtype, k) for k, v in flat_w.items()}
                a_in = {k: xl.graph_input(v.shape, v.dtype, k + "_acc", by_ref=True) for k, v in flat_a.items()}
                sin_i = xl.graph_input(sin.shape, sin.dtype, "sin")
                cos_i = xl.graph_input(cos.shape, cos.dtype, "cos")
                off_i = xl.graph_input((), xl.int32, "vocab_offset") if cfg.tp > 1 else None
                W = NamedTensors.from_dict(w_in)
                A = NamedTensors.from_dict(a_in)
                tok = ops.host_load(self.inputs.tokens)
                inp = ops.reshape(tok[:, :-1], (T,))
                lab = ops.reshape(tok[:, 1:], (T,))
                emb_call = emb_graph.bind(W.embedding).call_with_info(inp, *([off_i] if off_i is not None else []))
                x = emb_call.outputs[0]
                calls = []
                for i in range(cfg.layers):
                    info = blk_graph.bind(W.get(f"layer{i}")).call_with_info(x, sin_i, cos_i)
                    calls.append(info)
                    x = info.outputs[0]
                head_call = head_graph.bind(W.head).call_with_info(x)
                logits = head_call.outputs[0]
                if cfg.tp > 1:
                    loss, dlogits = cross_entropy_sharded_with_grad(logits, lab - off_i, 1.0,
                                                                    replica_grouping=par.tp_group)
                else:
                    loss, dlogits = ops.cross_entropy_with_grad(logits, lab, 1.0)
                ops.host_store(self.outputs.loss, ops.cast(loss, xl.float32))
                (dx,) = head_grad.bind(A.head).call(dlogits, args=head_grad.grad_graph_info.inputs_dict(head_call))
                for i in reversed(range(cfg.layers)):
                    (dx,) = blk_grad.bind(A.get(f"layer{i}")).call(
                        dx, args=blk_grad.grad_graph_info.inputs_dict(calls[i]))
                emb_grad.bind(A.embedding).call(dx, args=emb_grad.grad_graph_info.inputs_dict(emb_call))
            mb_inputs = {w_in[k]: flat_w[k] for k in flat_w}
            mb_inputs.update({a_in[k]: flat_a[k] for k in flat_a})
            mb_inputs[sin_i], mb_inputs[cos_i] = sin, cos
            if off_i is not None:
                mb_inputs[off_i] = offset_var
            ops.repeat(mb, self.micro_batches, inputs_dict=mb_inputs, cuda_graph=self.cuda_graphs)

            # ---- optimizer -------------------------------------------------------------------------------------
            groups = ([("embedding", emb_vars, emb_acc), ("head", head_vars, head_acc)] +
                      [(f"layer{i}", blk_vars[i], blk_acc[i]) for i in range(cfg.layers)])
            self.master, opt_state = build_optimizer(ir, cfg, par, groups, self.hp, self.state_dtype,
                                                     self.shard_optimizer, self.fused_collectives,
                                                     reduce_replicated_over=par.tp_group if cfg.sp else None)
            for atree in [emb_acc, head_acc] + blk_acc:
                ops.var_updates.accumulator_zero_(atree.mean_accum_counter)

        state = NamedTensors(model=weights)
        state.insert("master", NamedTensors.from_dict({k.replace(".", "_"): v for k, v in self.master.items()}))
        state.insert("adam", NamedTensors.from_dict({k.replace(".", "_"): v for k, v in opt_state.items()}))
        self.state = state
        self.weights = weights
        self.ir.num_host_transfers = self.micro_batches

    # ------------------------------------------------------------------------------------------------------------
    def step(self, tokens) -> float:
        """One optimizer step. `tokens`: int32 `(micro_batches, [replicas,] micro_batch_size, seq_len + 1)` on the
        host (pinned memory is used as is). Returns the mean loss of this rank's micro-batches."""
        out = self.session.run({self.inputs.tokens: tokens})
        return float(np.mean(out[self.outputs.loss]))

    def step_device(self, tokens_on_device: torch.Tensor) -> torch.Tensor:
        """As `step` for tokens already on the device; returns the per-micro-batch losses as a device tensor without
        synchronising (used to time the device work alone)."""
        out = self.session.run({self.inputs.tokens: tokens_on_device}, fetch=False)
        return out[self.outputs.loss]

    def synthetic_tokens(self, seed: int = 0, pinned: bool = True) -> torch.Tensor:
        """Uniform random token ids of the step's shape (what `step` expects for this process)."""
        g = torch.Generator().manual_seed(seed + int(os.environ.get("RANK", "0")) // max(self.cfg.tp, 1))
        local = 1 if self.session.distributed else self.cfg.tp * self.cfg.dp
        shape = (self.micro_batches, local, self.micro_batch_size, self.cfg.seq_len + 1)
        t = torch.randint(0, self.cfg.vocab_size, shape, generator=g, dtype=torch.int32)
        if not self.session.distributed and self.cfg.tp > 1:
            # replicas of one tensor-parallel group see the same data
            t = t[:, :: self.cfg.tp].repeat_interleave(self.cfg.tp, dim=1)
        if pinned and torch.cuda.is_available():
            t = t.pin_memory()
        return t
