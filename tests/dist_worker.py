"""Worker run under `torch.distributed.run` by the multi-process tests (CPU/gloo here, CUDA/NCCL on a GPU box).
Prints one JSON line from rank 0."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch


def global_tokens(cfg, micro_batches, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, cfg.vocab_size, (micro_batches, cfg.dp, 1, cfg.seq_len + 1), generator=g, dtype=torch.int32)
    return t.repeat_interleave(cfg.tp, dim=1)  # replicas of one tensor-parallel group see the same data


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="train")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=2)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--fused", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--big", type=int, default=0)
    ap.add_argument("--gemm-m", dest="m", type=int, default=2048)
    ap.add_argument("--gemm-n", dest="n", type=int, default=4096)
    ap.add_argument("--gemm-k", dest="k", type=int, default=4096)
    ap.add_argument("--n-copy", type=int, default=16)
    ap.add_argument("--n-red", type=int, default=8)
    ap.add_argument("--slots", type=int, default=2)
    ap.add_argument("--ckpt", default="")
    ap.add_argument("--sp", type=int, default=0)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    import torch.distributed as dist

    if args.mode == "train":
        from popxl_addons_b200.models.decoder import DecoderConfig
        from popxl_addons_b200.models.gptj import GPTJConfig
        from popxl_addons_b200.models.trainer import DecoderTrainer

        cfg = (GPTJConfig.tiny(dtype=args.dtype, tp=args.tp, dp=args.dp, **({"seq_len": 512} if args.big == 2 else {}))
               if args.big else DecoderConfig.tiny("gptj", dtype=args.dtype, tp=args.tp, dp=args.dp))
        cfg.sequence_parallel = bool(args.sp)
        if args.device == "cuda":
            from popxl_addons_b200.ops import native

            native.STRICT[0] = True  # a hot op that runs its torch implementation on the GPU is an error
        trainer = DecoderTrainer(cfg, micro_batches=2, device=args.device, lr=1e-2 if args.big < 2 else 2e-3,
                                 fused_collectives=bool(args.fused))
        losses = []
        for step in range(args.steps):
            tok = global_tokens(cfg, 2, seed=step)
            if world > 1:
                tok = tok[:, rank:rank + 1]
            loss = torch.tensor([trainer.step(tok)], dtype=torch.float64, device=trainer.session.device)
            if world > 1:
                dist.all_reduce(loss)  # mean over all replicas, like the in-process simulation reports
                loss /= world
            losses.append(float(loss))
        w = trainer.session.get_tensor_data(trainer.weights.layer0.get("mlp.fc_in.weight"))
        extra = {}
        if args.device == "cuda":
            from popxl_addons_b200.ops import native

            extra["kernels"] = native.LAUNCHES["by_kernel"]
            extra["fallbacks"] = dict(native.FALLBACKS)
        if rank == 0:
            print(json.dumps({"losses": losses, "w_sum": float(np.abs(w).sum()), "fused_pairs":
                              trainer.fused_gemm_collectives, **extra}))
    elif args.mode == "collectives":
        # every collective of the communicator against a closed form
        from popxl_addons_b200 import xl as popxl
        from popxl_addons_b200.xl import ops
        import popxl_addons_b200 as addons

        ir = popxl.Ir(replication="popdist")
        with ir.main_graph:
            h2d = popxl.h2d_stream((6,), popxl.float32)
            x = ops.host_load(h2d)
            grp = ir.replica_grouping()
            ar = ops.collectives.replicated_all_reduce(x, "add", grp)
            mx = ops.collectives.replicated_all_reduce(x, "max", grp)
            rs = ops.collectives.replicated_reduce_scatter(x, "mean", grp)
            ag = ops.collectives.replicated_all_gather(rs, grp)
            streams = [addons.host_store(t) for t in (ar, mx, rs, ag)]
        s = popxl.Session(ir, args.device)
        data = np.arange(6 * world, dtype=np.float32).reshape(world, 6)
        out = s.run({h2d: data[rank]})
        ok = bool(np.allclose(out[streams[0]], data.sum(0)) and np.allclose(out[streams[1]], data.max(0))
                  and np.allclose(out[streams[3]], data.mean(0)))
        n = 6 // world
        ok = ok and bool(np.allclose(out[streams[2]], data.mean(0)[rank * n:(rank + 1) * n]))
        # hidden-sharded LayerNorm (native kernels + one small all-reduce on the GPU) against the full-width LayerNorm
        from popxl_addons_b200.ops.layer_norm_distributed import layer_norm_distributed

        rs = np.random.RandomState(7)
        full = rs.normal(size=(5, 16 * world)).astype(np.float32)
        gamma, beta = rs.normal(size=16 * world).astype(np.float32), rs.normal(size=16 * world).astype(np.float32)
        ir2 = popxl.Ir(replication="popdist")
        with ir2.main_graph:
            hx = popxl.h2d_stream((5, 16), popxl.float32)
            hw, hb = popxl.h2d_stream((16,), popxl.float32), popxl.h2d_stream((16,), popxl.float32)
            y = layer_norm_distributed(ops.host_load(hx), ops.host_load(hw), ops.host_load(hb), 1e-5,
                                       ir2.replica_grouping())
            out_y = addons.host_store(y)
        s2 = popxl.Session(ir2, args.device)
        sl = slice(16 * rank, 16 * (rank + 1))
        got = s2.run({hx: full[:, sl], hw: gamma[sl], hb: beta[sl]})[out_y]
        mu, var = full.mean(-1, keepdims=True), full.var(-1, keepdims=True)
        want = ((full - mu) / np.sqrt(var + 1e-5) * gamma + beta)[:, sl]
        ok = ok and bool(np.allclose(got, want, rtol=1e-4, atol=1e-4))
        flag = torch.tensor([int(ok)], device=s.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({"ok": bool(flag.item())}))
    elif args.mode == "fusedgemm":
        # GEMM + reduce-scatter and all-gather + GEMM kernels against NCCL + torch.matmul on the same data
        from popxl_addons_b200 import xl as popxl
        from popxl_addons_b200.ops import native
        from popxl_addons_b200.parallel import fused

        ir = popxl.Ir(replication="popdist")
        with ir.main_graph:
            pass
        s = popxl.Session(ir, "cuda")
        fused.runtime(s).reserve(ir.replica_grouping(), 640 << 20)  # operands of the micro-benchmarks below
        ctx = fused.runtime(s).context(ir.replica_grouping())
        dev = s.device
        M, N, K = args.m, args.n, args.k
        result = {"world": world}

        def timed(fn, iters=10):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record()
            for _ in range(iters):
                fn()
            en.record()
            torch.cuda.synchronize()
            t = torch.tensor([st.elapsed_time(en) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        torch.manual_seed(100 + rank)
        # --- reduce-scatter: every rank holds a K-slice of the contraction -------------------------------------------
        a = (torch.randn(M, K, device=dev) * 0.1).bfloat16()
        w = (torch.randn(K, N, device=dev) * 0.1).bfloat16()
        full = a.float() @ w.float()
        dist.all_reduce(full)
        mine = fused.gemm_reduce_scatter(ctx, a, w)
        assert mine is not NotImplemented
        torch.cuda.synchronize()
        want = full[rank * (M // world):(rank + 1) * (M // world)]
        result["rs_err"] = float((mine.float() - want).abs().max() / want.abs().max())
        result["rs_ms"] = timed(lambda: fused.gemm_reduce_scatter(ctx, a, w))

        def nccl_rs():
            y = a @ w
            out = torch.empty(M // world, N, device=dev, dtype=y.dtype)
            dist.reduce_scatter_tensor(out, y)
            return out

        result["rs_nccl_ms"] = timed(nccl_rs)
        result["gemm_ms"] = timed(lambda: native.gemm(a, w))

        # GEMM + all-reduce: multimem.red epilogue (zero + kernel + copy out, as the graph op does) vs GEMM + NCCL
        def fused_ar():
            out = ctx.arena.ring((M, N), a.dtype)
            out.zero_()
            native.gemm(a, w, out=out, accumulate=3, comm=ctx)
            return out.clone()

        def nccl_ar():
            y = native.gemm(a, w)
            dist.all_reduce(y)
            return y

        got = fused_ar()
        torch.cuda.synchronize()
        result["ar_err"] = float((got.float() - full).abs().max() / full.abs().max())
        result["ar_fused_ms"] = timed(fused_ar)
        result["ar_nccl_ms"] = timed(nccl_ar)
        # GEMM + all-reduce by pulling: partial tiles stay local, NVSwitch adds them on the way into the owner of the rows
        got = fused.gemm_all_reduce_pull(ctx, [(a, w)], n_red=args.n_red)
        assert got is not NotImplemented
        got = got.clone()
        torch.cuda.synchronize()
        result["ar_pull_err"] = float((got.float() - full).abs().max() / full.abs().max())
        result["ar_pull_ms"] = timed(lambda: fused.gemm_all_reduce_pull(ctx, [(a, w)], n_red=args.n_red))
        # where the time of the pulling kernel goes: per-CTA timestamps of one launch (start, tiles done, reduce work
        # done, checked in), relative to the earliest start, in microseconds
        bn = 128 if os.environ.get("XL_AR_PULL_BLOCK_N") == "128" else 256
        n_items = (M // ctx.world // 128) * ((N + bn - 1) // bn) * 8
        stamps = torch.zeros((148 + n_items) * 4, dtype=torch.int64, device=dev)
        for it in range(4):  # launches close with a barrier over the ranks: the last one starts on all ranks together
            fused.gemm_all_reduce_pull(ctx, [(a, w)], n_red=args.n_red, timestamps=stamps if it == 3 else None)
        torch.cuda.synchronize()
        if os.environ.get("XL_DUMP_TIMELINE"):
            np.save(f"{os.environ['XL_DUMP_TIMELINE']}_rank{ctx.rank}.npy", stamps.cpu().numpy())
        st = stamps[:148 * 4].view(148, 4).cpu().numpy().astype(np.int64)
        used = st[:, 0] > 0
        t0 = st[used, 0].min()
        rel = (st[used] - t0) / 1e3
        red = rel[:args.n_red]
        gem = rel[args.n_red:]
        items = stamps[148 * 4:].view(n_items, 4).cpu().numpy().astype(np.int64)
        items = (items[items[:, 0] > 0, :3] - t0) / 1e3
        wait, work = items[:, 1] - items[:, 0], items[:, 2] - items[:, 1]
        result["pull_items_us"] = {"n": int(len(items)), "taken": [float(items[:, 0].min()), float(np.median(items[:, 0])), float(items[:, 0].max())],
                                   "wait_for_tile": [float(np.median(wait)), float(wait.max())],
                                   "reduce": [float(work.min()), float(np.median(work)), float(work.max())],
                                   "last_done": float(items[:, 2].max())}
        result["pull_timeline_us"] = {
            "reducer_ctas": {"reduce_done": [float(red[:, 2].min()), float(red[:, 2].max())],
                             "finish": [float(red[:, 3].min()), float(red[:, 3].max())]},
            "gemm_ctas": {"start": [float(gem[:, 0].min()), float(gem[:, 0].max())],
                          "tiles_done": [float(gem[:, 1].min()), float(np.median(gem[:, 1])), float(gem[:, 1].max())],
                          "reduce_done": [float(gem[:, 2].min()), float(np.median(gem[:, 2])), float(gem[:, 2].max())],
                          "finish": [float(gem[:, 3].min()), float(gem[:, 3].max())]}}
        # two operand pairs contracted into one accumulator: all_reduce(a @ w + a2 @ w2), K2 = K / 4 (a block's attention
        # and feed-forward output projections), and the transposed-weight form of the backward pass
        K2 = max(64, K // 4)
        a2 = (torch.randn(M, K2, device=dev) * 0.1).bfloat16()
        w2 = (torch.randn(K2, N, device=dev) * 0.1).bfloat16()
        full2 = a.float() @ w.float() + a2.float() @ w2.float()
        dist.all_reduce(full2)
        got = fused.gemm_all_reduce_pull(ctx, [(a, w), (a2, w2)], n_red=args.n_red)
        assert got is not NotImplemented
        got = got.clone()
        torch.cuda.synchronize()
        result["ar_pull2_err"] = float((got.float() - full2).abs().max() / full2.abs().max())
        result["ar_pull2_ms"] = timed(lambda: fused.gemm_all_reduce_pull(ctx, [(a, w), (a2, w2)], n_red=args.n_red))
        wt, w2t = w.t().contiguous(), w2.t().contiguous()  # stored (N, K): K-major right operands, as in a data gradient
        got = fused.gemm_all_reduce_pull(ctx, [(a, wt.t()), (a2, w2t.t())], n_red=args.n_red)
        assert got is not NotImplemented
        got = got.clone()
        torch.cuda.synchronize()
        result["ar_pull2_t_err"] = float((got.float() - full2).abs().max() / full2.abs().max())
        for _ in range(20):  # many launches back to back: the flag words and the work queue must come back to zero
            got = fused.gemm_all_reduce_pull(ctx, [(a, w), (a2, w2)], n_red=args.n_red)
        got = got.clone()
        torch.cuda.synchronize()
        result["ar_pull2_repeat_err"] = float((got.float() - full2).abs().max() / full2.abs().max())

        # reduce-scatter by pulling (the owner keeps the sums) and all-gather by multicast
        mine2 = fused.gemm_reduce_scatter_pull(ctx, [(a, w), (a2, w2)], n_red=args.n_red)
        assert mine2 is not NotImplemented
        torch.cuda.synchronize()
        want2 = full2[rank * (M // world):(rank + 1) * (M // world)]
        result["rs_pull2_err"] = float((mine2.float() - want2).abs().max() / want2.abs().max())
        result["rs_pull2_ms"] = timed(lambda: fused.gemm_reduce_scatter_pull(ctx, [(a, w), (a2, w2)], n_red=args.n_red))
        shard_rows = (torch.randn(M // world, N, device=dev) * 0.1).bfloat16()
        gathered_ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gathered_ref, shard_rows)
        got = fused.all_gather_multicast(ctx, shard_rows)
        assert got is not None
        torch.cuda.synchronize()
        result["ag_mc_ok"] = bool(torch.equal(got, gathered_ref))
        for _ in range(9):  # the ring of two buffers and the barrier channel, many calls back to back
            got = fused.all_gather_multicast(ctx, shard_rows)
        torch.cuda.synchronize()
        result["ag_mc_repeat_ok"] = bool(torch.equal(got, gathered_ref))
        result["ag_mc_ms"] = timed(lambda: fused.all_gather_multicast(ctx, shard_rows))
        result["ag_nccl_ms"] = timed(lambda: dist.all_gather_into_tensor(gathered_ref, shard_rows))

        def nccl_ar2():
            y = native.gemm(a, w)
            native.gemm(a2, w2, out=y, accumulate=1)
            dist.all_reduce(y)
            return y

        def cublas_ar2():
            y = torch.addmm(a @ w, a2, w2)
            dist.all_reduce(y)
            return y

        result["ar_nccl2_ms"] = timed(nccl_ar2)
        result["ar_cublas_nccl2_ms"] = timed(cublas_ar2)
        result["gemm2_ms"] = timed(lambda: native.gemm(a2, w2, out=native.gemm(a, w), accumulate=1))
        ybuf = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        result["nccl_all_reduce_only_ms"] = timed(lambda: dist.all_reduce(ybuf))
        small = torch.randn(2048, device=dev)
        result["small_all_reduce_ms"] = timed(lambda: s.comm.all_reduce([small], ir.replica_grouping(), "add"))
        act = torch.randn(16, 4096, device=dev).bfloat16()
        result["mc_all_reduce_16x4096_ms"] = timed(lambda: s.comm.all_reduce([act], ir.replica_grouping(), "add"))
        result["nccl_all_reduce_16x4096_ms"] = timed(lambda: dist.all_reduce(act))
        # --- all-gather of the left operand (rows sharded) ---------------------------------------------------------------
        a_full, a_own = fused.gathered_operand(ctx, M, K, torch.bfloat16, 128, "a")
        a_own.copy_((torch.randn(M // world, K, device=dev) * 0.1).bfloat16())
        gathered = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gathered, a_own.contiguous())
        # poison the remote rows so that stale data cannot pass
        for r in range(world):
            if r != rank:
                a_full[r * (M // world):(r + 1) * (M // world)].fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        y = fused.all_gather_gemm(ctx, a_full, w, sharded="a", n_copy=args.n_copy)
        assert y is not NotImplemented
        torch.cuda.synchronize()
        want = gathered.float() @ w.float()
        result["ag_a_err"] = float((y.float() - want).abs().max() / want.abs().max())
        result["ag_a_gathered_ok"] = bool(torch.equal(a_full, gathered))
        result["ag_a_ms"] = timed(lambda: fused.all_gather_gemm(ctx, a_full, w, sharded="a", n_copy=args.n_copy))

        def nccl_ag():
            g = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            dist.all_gather_into_tensor(g, a_own)
            return g @ w

        result["ag_a_nccl_ms"] = timed(nccl_ag)
        # --- all-gather of the right operand (a weight whose K rows are sharded) -------------------------------------------
        w_full, w_own = fused.gathered_operand(ctx, K, N, torch.bfloat16, 64, "w")
        w_own.copy_((torch.randn(K // world, N, device=dev) * 0.1).bfloat16())
        wg = torch.empty(K, N, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(wg, w_own.contiguous())
        for r in range(world):
            if r != rank:
                w_full[r * (K // world):(r + 1) * (K // world)].fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        y = fused.all_gather_gemm(ctx, a, w_full, sharded="b", n_copy=args.n_copy)
        assert y is not NotImplemented
        torch.cuda.synchronize()
        want = a.float() @ wg.float()
        result["ag_b_err"] = float((y.float() - want).abs().max() / want.abs().max())
        result["ag_b_gathered_ok"] = bool(torch.equal(w_full, wg))
        result["ag_b_ms"] = timed(lambda: fused.all_gather_gemm(ctx, a, w_full, sharded="b", n_copy=args.n_copy))
        # --- decode step: all-reduce + residual + LayerNorm in one kernel vs NCCL + the local kernel -----------------------------
        from types import SimpleNamespace

        xr = torch.randn(16, 4096, device=dev).bfloat16()
        dl = (torch.randn(16, 4096, device=dev) * 0.5).bfloat16()
        bs = torch.randn(4096, device=dev).bfloat16()
        lw, lb = torch.randn(4096, device=dev).bfloat16(), torch.randn(4096, device=dev).bfloat16()
        dist.broadcast(xr, 0)  # the residual stream is identical on the ranks of a TP group
        for t_ in (bs, lw, lb):
            dist.broadcast(t_, 0)
        fake_op = SimpleNamespace(attrs=dict(group=ir.replica_grouping(), has_bias=True, eps=1e-5))
        for trial in range(3):  # several calls: the staging halves alternate
            x1, x2 = xr.clone(), xr.clone()
            (h1,) = fused.ar_add_layer_norm(s, fake_op, [x1], [dl], [bs], [lw], [lb])
            dsum = dl.float().clone()
            dist.all_reduce(dsum)
            h2 = native.add_layer_norm_cuda(x2, dsum.bfloat16(), bs, lw, lb, has_delta=True, has_bias=True, eps=1e-5)
            torch.cuda.synchronize()
            result["ar_ln_err"] = max(result.get("ar_ln_err", 0.0), float((h1.float() - h2.float()).abs().max()),
                                      float((x1.float() - x2.float()).abs().max()))
        x1 = xr.clone()
        result["ar_ln_fused_ms"] = timed(lambda: fused.ar_add_layer_norm(s, fake_op, [x1], [dl], [bs], [lw], [lb]))

        def nccl_ar_ln():
            d = dl.clone()
            dist.all_reduce(d)
            return native.add_layer_norm_cuda(x1, d, bs, lw, lb, has_delta=True, has_bias=True, eps=1e-5)

        result["ar_ln_nccl_ms"] = timed(nccl_ar_ln)
        # --- fused reduce-scatter + AdamW + all-gather over peer pointers (one kernel) vs NCCL + the local Adam kernel --------
        import ctypes

        n_par = 1 << 26  # 64 Mi parameters
        shard = n_par // world
        wt = ctx.arena.alloc((n_par,), torch.bfloat16)
        acc = ctx.arena.alloc((n_par,), torch.float32)
        wt.normal_(0, 0.02)
        acc.normal_(0, 1e-3)
        master = wt[rank * shard:(rank + 1) * shard].float()
        m1, v1 = torch.zeros_like(master), torch.zeros_like(master)
        step_t = torch.zeros((), device=dev)
        grads = (ctypes.c_void_p * world)(*ctx.arena.peer_ptrs(acc))
        weights = (ctypes.c_void_p * world)(*ctx.arena.peer_ptrs(wt))
        torch.cuda.synchronize()
        dist.barrier()

        def fused_adam():
            fused.group_barrier(ctx, 4)
            native._check(native._rts_adam(grads, weights, native._CODE[wt.dtype], master.data_ptr(), m1.data_ptr(),
                                           native._CODE[m1.dtype], v1.data_ptr(), step_t.data_ptr(), rank * shard, shard,
                                           world, 1e-4, 0.9, 0.95, 1e-5, 0.01, 1.0, 1, native._stream()), "rts_adam")
            fused.group_barrier(ctx, 5)

        g_shard = torch.empty(shard, device=dev)
        w_full = torch.empty(n_par, device=dev, dtype=torch.bfloat16)

        def nccl_adam():
            dist.reduce_scatter_tensor(g_shard, acc, op=dist.ReduceOp.AVG)
            native.adam_cuda(w_full[rank * shard:(rank + 1) * shard], g_shard, m1, v1, step_t, master, has_step=True,
                             has_master=True, bias_correction=True, lr=1e-4, beta1=0.9, beta2=0.95, epsilon=1e-5,
                             weight_decay=0.01, grad_scale=1.0, _tensor_scalars=())
            dist.all_gather_into_tensor(w_full, w_full[rank * shard:(rank + 1) * shard].clone())

        result["rts_adam_fused_ms"] = timed(fused_adam, iters=5)
        result["rts_adam_nccl_ms"] = timed(nccl_adam, iters=5)
        result["rts_adam_params"] = n_par
        try:
            ctx.check()
            native.check_gemm_errors()
            result["errors"] = None
        except Exception as e:  # a bounded wait gave up
            result["errors"] = str(e)
        result["shape"] = [M, N, K]
        if rank == 0:
            print(json.dumps(result))
    elif args.mode == "pipeline":
        # a replica spans `--slots` processes: forward on slot 0, loss term on slot 1, backward on slot 0 again;
        # stage boundaries are send/recv between the processes, replicas are data-parallel (gradient all-reduce)
        from popxl_addons_b200 import xl as popxl
        from popxl_addons_b200.xl import ops
        import popxl_addons_b200 as addons
        from popxl_addons_b200.layers import Linear

        steps, slots = 6, args.slots
        np.random.seed(42)
        ir = popxl.Ir(replication="popdist", devices_per_replica=slots)
        R = ir.replication_factor
        data = np.random.normal(0, 1, (steps, R, 1, 4)).astype(np.float32)
        with ir.main_graph:
            with addons.pipelined_execution(steps) as p:
                with p.stage(0), popxl.ipu(0):
                    _, x_stream, x = addons.host_load(data[0, 0], popxl.float32, "x")
                    fargs, lin = Linear(4).create_graph(x)
                    dargs, dlin = addons.autodiff_with_accumulation(lin, [lin.args.weight])
                    w, dw = fargs.init(), dargs.init()
                    info = lin.bind(w).call_with_info(x)
                    y, *_ = info.outputs
                    y = y.copy_to_ipu(1)
                with p.stage(1), popxl.ipu(1):
                    scale = popxl.variable(np.full((4,), 2.0, np.float32), name="scale")
                    y = y * scale + 1
                    y = y.copy_to_ipu(0)
                with p.stage(2), popxl.ipu(0):
                    dlin.bind(dw).call(y, args=p.stash_and_restore_activations(info, dlin.grad_graph_info))
            with popxl.ipu(0):
                g = ops.collectives.replicated_all_reduce(dw.accum.weight, "mean", ir.replica_grouping())
                out = addons.host_store(g)
        ir.num_host_transfers = steps
        s = popxl.Session(ir, args.device)
        replica, slot = rank // slots, rank % slots
        res = s.run({x_stream: data[:, replica]})
        owned = {"w": s.owns(w.weight), "dw": s.owns(dw.accum.weight), "scale": s.owns(scale)}
        payload = {"rank": rank, "slot": slot, "owned": owned}
        if slot == 0:
            payload["grad"] = np.asarray(res[out]).reshape(-1).tolist()
        gathered = [None] * world
        dist.all_gather_object(gathered, payload)
        if rank == 0:
            print(json.dumps({"ranks": gathered, "data_seed": 42}))
    elif args.mode == "pp_train":
        # pipeline-parallel trainer: `--slots` processes per replica, world / slots data-parallel replicas
        from popxl_addons_b200.models import decoder as dec
        from popxl_addons_b200.models.decoder import DecoderConfig
        from popxl_addons_b200.models.pipeline_trainer import PipelineTrainer

        dp = world // args.slots
        cfg = DecoderConfig.tiny("llama", layers=4, dtype=args.dtype, tp=1, dp=dp)
        dec._SEED[0] = 0
        tr = PipelineTrainer(cfg, stages=args.slots, micro_batches=6, device=args.device, lr=1e-2,
                             fused_collectives=bool(args.fused))
        replica = rank // args.slots
        losses = []
        for step in range(args.steps):
            g = torch.Generator().manual_seed(step)
            tok = torch.randint(0, cfg.vocab_size, (6, dp, 1, cfg.seq_len + 1), generator=g, dtype=torch.int32)
            loss = tr.step(tok[:, replica:replica + 1])
            losses.append(loss)
        ckpt_ok = None
        if args.ckpt:
            # every process writes the variables of its own device slot into one directory and restores them from it
            sess = tr.session
            before = {k: v.copy() for k, v in sess.get_named_tensors_data().to_dict().items()}
            sess.save_checkpoint(args.ckpt)  # returns once every slot's files and the completion marker are written
            assert os.path.exists(os.path.join(args.ckpt, "session_info.json"))
            for var in sess._owned_state().values():
                sess.write_variable_data(var, np.zeros(var.shape_on_host, dtype=np.float32))
            sess.load_checkpoint(args.ckpt, report_missing="error")
            after = sess.get_named_tensors_data().to_dict()
            ckpt_ok = bool(set(before) == set(after) and all(np.array_equal(before[k], after[k]) for k in before))
        gathered = [None] * world
        dist.all_gather_object(gathered, {"rank": rank, "losses": losses, "ckpt_ok": ckpt_ok,
                                          "n_owned": len(tr.session._owned_state())})
        if rank == 0:
            print(json.dumps({"ranks": gathered, "n_state": len(tr.state.to_dict())}))
    elif args.mode == "rtsclip":
        # bucketed RTS optimizer on the device: (a) one fused launch per bucket, (b) reduce + global norm + clipped update,
        # both against a numpy AdamW on the averaged gradients
        from popxl_addons_b200 import xl as popxl
        from popxl_addons_b200.xl import ops
        if args.device == "cuda":
            from popxl_addons_b200.ops import native
        from popxl_addons_b200.optimizers.rts_adam import rts_adam_bucket_, rts_reduce_bucket_

        shapes, decays, lr, max_norm = [(256, 192), (4096,), (512, 64)], (0.01, 0.0, 0.01), 1e-2, 0.5
        rs = np.random.RandomState(3)
        w0 = [rs.randn(*sh).astype(np.float32) * 0.1 for sh in shapes]
        w0 = [torch.tensor(w).bfloat16().float().numpy() for w in w0]
        grads = [[rs.randn(*sh).astype(np.float32) for sh in shapes] for _ in range(world)]
        mean_g = [np.mean([grads[r][k] for r in range(world)], axis=0) for k in range(len(shapes))]
        norm = float(np.sqrt(sum((g.astype(np.float64) ** 2).sum() for g in mean_g)))

        def adamw(w, g, decay, scale):
            g = g * scale
            m, v = 0.1 * g, 0.05 * g * g
            upd = (m / (1 - 0.9)) / (np.sqrt(v / (1 - 0.95)) + 1e-5) + w * decay
            return w - lr * upd

        results = {}
        for clip in (False, True):
            ir = popxl.Ir(replication="popdist")
            with ir.main_graph:
                rg = ir.replica_grouping()
                one = ir.replica_grouping(group_size=1)
                ws, accs, masters, ms, vs = [], [], [], [], []
                for k, sh in enumerate(shapes):
                    w = popxl.variable(w0[k], popxl.bfloat16, f"w{k}")
                    acc = popxl.variable(np.stack([grads[r][k] for r in range(world)]), popxl.float32, f"acc{k}",
                                         replica_grouping=one)
                    w.symmetric_group = rg
                    acc.symmetric_group = rg
                    master, _ = popxl.replica_sharded_variable(w0[k], popxl.float32, f"master{k}", shard_grouping=rg)
                    m, _ = popxl.replica_sharded_variable(np.zeros(sh, np.float32), popxl.float32, f"m{k}", shard_grouping=rg)
                    v, _ = popxl.replica_sharded_variable(np.zeros(sh, np.float32), popxl.float32, f"v{k}", shard_grouping=rg)
                    ws.append(w), accs.append(acc), masters.append(master), ms.append(m), vs.append(v)
                step = popxl.variable(np.zeros((), np.float32), popxl.float32, "step")
                if clip:
                    sumsq = rts_reduce_bucket_(accs, rg)
                    total = ops.collectives.replicated_all_reduce(sumsq, "add", rg)
                    gmax = popxl.constant(max_norm, popxl.float32)
                    factor = ops.div(gmax, ops.maximum(ops.sqrt(total), gmax))
                    rts_adam_bucket_(ws, accs, masters, ms, vs, step, rg, lr=lr, weight_decays=decays, beta1=0.9, beta2=0.95,
                                     eps=1e-5, scale=factor, reduced=True)
                else:
                    rts_adam_bucket_(ws, accs, masters, ms, vs, step, rg, lr=lr, weight_decays=decays, beta1=0.9, beta2=0.95,
                                     eps=1e-5)
            sess = popxl.Session(ir, args.device)
            sess.run()
            scale = min(1.0, max_norm / norm) if clip else 1.0
            err = 0.0
            for k in range(len(shapes)):
                got = sess.get_tensor_data(ws[k]).astype(np.float32)
                want = adamw(w0[k], mean_g[k], decays[k], scale)
                err = max(err, float(np.abs(got - want).max() / np.abs(want).max()))
                mgot = sess.get_tensor_data(masters[k])
                err = max(err, 10 * float(np.abs(mgot - want).max() / np.abs(want).max()))  # fp32 master: 10x tighter
            results["clip" if clip else "fused"] = err
        if rank == 0:
            print(json.dumps({"errors": results, "norm": norm,
                              "kernels": native.LAUNCHES["by_kernel"] if args.device == "cuda" else {}}))
    elif args.mode == "elastic":
        # data-parallel training under the restart supervisor: checkpoints every 2 steps, heartbeats between steps; on
        # the first attempt rank 1 stops after step 3 (a host-side failure, nothing in flight)
        from popxl_addons_b200.models import decoder as dec
        from popxl_addons_b200.models.decoder import DecoderConfig
        from popxl_addons_b200.models.trainer import DecoderTrainer
        from popxl_addons_b200.parallel.elastic import latest_checkpoint
        from popxl_addons_b200.parallel.health import Heartbeat, PeerLost

        attempt = int(os.environ.get("XL_RESTART_COUNT", "0"))
        inject = os.environ.get("XL_TEST_INJECT_FAILURE") == "1" and attempt == 0
        dec._SEED[0] = 0
        cfg = DecoderConfig.tiny("gptj", dtype="float32", tp=1, dp=world)
        trainer = DecoderTrainer(cfg, micro_batches=2, device="cpu", lr=1e-2)
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world)
        start = 0
        ck = latest_checkpoint(args.ckpt)
        if ck is not None:
            trainer.session.load_checkpoint(ck, report_missing="error")
            start = int(trainer.session.session_state["steps"])
        losses = {}
        try:
            for step in range(start, args.steps):
                if step > start:
                    hb.check_peers(step - 1, timeout=20.0)
                losses[step] = trainer.step(global_tokens(cfg, 2, seed=step)[:, rank:rank + 1])
                if inject and rank == 1 and step == 3:
                    hb.beat(step, "failed")
                    os._exit(7)
                hb.beat(step)
                if (step + 1) % 2 == 0:
                    hb.check_peers(step, timeout=20.0)  # the checkpoint gathers over all ranks
                    trainer.session.save_checkpoint(os.path.join(args.ckpt, f"step{step + 1}"))
        except PeerLost:
            os._exit(3)
        w = trainer.session.get_tensor_data(trainer.weights.layer0.get("mlp.fc_in.weight"))
        if rank == 0:
            with open(os.path.join(args.ckpt, "result.json"), "w") as f:
                json.dump({"attempt": attempt, "resumed_from": start, "losses": losses,
                           "w": np.asarray(w, np.float64).ravel()[:64].tolist(), "w_sum": float(np.abs(w).sum()),
                           "steps": int(trainer.session.session_state["steps"])}, f)
        dist.barrier()
        os._exit(0)
    elif args.mode == "fail":
        # rank 1 stops between steps; rank 0 notices on the host before launching anything that would wait for it
        from datetime import timedelta

        from popxl_addons_b200.parallel.health import Heartbeat, PeerLost

        dist.init_process_group("gloo", timeout=timedelta(seconds=20))
        store = dist.distributed_c10d._get_default_store()
        hb = Heartbeat(store, rank, world)
        result = {"detected": False}
        for step in range(3):
            try:
                hb.check_peers(step - 1, timeout=3.0)
            except PeerLost as e:
                result = {"detected": True, "missing": e.missing, "step": step}
                break
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            if rank == 1 and step == 1:
                hb.beat(step, "failed")
                os._exit(0)  # leaves between steps, nothing in flight
            hb.beat(step)
        if rank == 0:
            print(json.dumps(result))
        os._exit(0)
    if dist.is_initialized():
        dist.barrier()
        if args.device == "cuda":
            # leave without tearing NCCL down: with captured CUDA graphs alive that has been seen to block for minutes
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
