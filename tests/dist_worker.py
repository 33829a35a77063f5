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

        cfg = (GPTJConfig.tiny(dtype=args.dtype, tp=args.tp, dp=args.dp) if args.big
               else DecoderConfig.tiny("gptj", dtype=args.dtype, tp=args.tp, dp=args.dp))
        trainer = DecoderTrainer(cfg, micro_batches=2, device=args.device, lr=1e-2,
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
        flag = torch.tensor([int(ok)], device=s.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({"ok": bool(flag.item())}))
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
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
