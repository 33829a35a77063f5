"""Headline benchmark: training throughput (tokens/s) of a GPT-J-6B-shape decoder, bf16 compute with fp32 master
weights and fp32 Adam state, sequence length 2048, 16 micro-batches of 1 sequence per data-parallel replica and step,
tensor parallel x data parallel with the optimizer state sharded over the data-parallel group (TP4 x DP2 on 8 GPUs).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model gptj_6b|gpt2_small|llama2_7b]

With N > 1 it is launched by `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...` (one rank per
GPU). Rank 0 prints one JSON line. `value` is timed on the device with CUDA events around K steps whose inputs are
already resident; `e2e` is timed around the public `DecoderTrainer.step` call, which copies each step's tokens from
pinned host memory and reads the losses back.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "train tokens/s GPT-J-6B shape TPxDP (bf16, fp32 Adam, seq 2048, 16 micro-batches of 1)"


def layout_for(n_gpus: int):
    tp = min(n_gpus, 4)
    return tp, n_gpus // tp


class ClockSampler:
    """Polls nvidia-smi while the timed region runs (SM clock and throttle reasons of this rank's GPU)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        sm = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def run_reference(args):
    """Runs the unmodified reference from `baseline/_ref` if it can be imported. It needs Graphcore's Poplar SDK
    (`popxl`, `popart`) and an IPU, so on this platform the import fails and the arm reports itself unavailable."""
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "popxl_addons")):
        why = "baseline/_ref/popxl_addons is not installed"
    else:
        sys.path.insert(0, ref)
        try:
            import popxl_addons  # noqa: F401
        except Exception as e:  # ModuleNotFoundError: No module named 'popxl'
            why = (f"`import popxl_addons` from baseline/_ref fails with {type(e).__name__}: {e} "
                   "(the reference is a layer on Graphcore's Poplar SDK, which exists only for IPU systems)")
    if why is None:
        why = "the reference imported, but it can only execute on Graphcore IPU hardware (popxl.Session needs an IPU)"
    if int(os.environ.get("RANK", "0")) == 0:  # one line per job, also when launched with one process per GPU
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


PIPELINE_METRIC = "train tokens/s Llama-2-7B shape PPxDP (bf16, fp32 Adam, seq 2048, 32 micro-batches of 1)"
DECODE_METRIC = "int4 decode tokens/s GPT-J-6B shape, TP over all GPUs (batch 16, prompt 512, 128 new tokens, greedy)"


def _shrink(cfg, k: int):
    """One rank's share of a k-way tensor-parallel layout as a stand-alone model (diagnostics only)."""
    cfg.heads //= k
    cfg.ffn //= k
    cfg.vocab_size = (cfg.vocab_size + k - 1) // k


def _shutdown(dist):
    """Leave without tearing the NCCL communicators down: destroying them while captured CUDA graphs that contain
    their kernels are still alive has been seen to block for minutes."""
    if dist is not None:
        dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    if dist is not None:
        os._exit(0)


def run_decode(args):
    """Int4 group-quantised greedy generation: weights N(0, 0.02) quantised in groups of 64 along the input dimension
    with fp16 scale and bias, bf16 activations and KV cache, tensor parallel over all GPUs. One step = one whole
    `generate` call (prefill of the prompts + `new_tokens - 1` single-token steps)."""
    import numpy as np
    import torch

    from popxl_addons_b200.models.decoder import DecoderConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    cfg = getattr(DecoderConfig, args.model)(tp=args.gpus, dp=1)
    if args.layers:
        cfg.layers = args.layers
    if args.emulate_tp:
        _shrink(cfg, args.emulate_tp)
    W, K = max(args.warmup, 3), args.steps
    B, P, N = args.batch, args.prompt_len, args.new_tokens
    t0 = time.perf_counter()
    if args.impl == "torch":
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        from torch_generator import TorchGenerator

        gen = TorchGenerator(cfg, B, P, N, group_size=64, cache_dense=args.torch_dense,
                             cuda_graph=not args.no_cuda_graphs)
        launches_of = lambda: 0  # noqa: E731
        kernels_of = lambda: {}  # noqa: E731
    else:
        from popxl_addons_b200.models.generator import DecoderGenerator
        from popxl_addons_b200.ops import native

        gen = DecoderGenerator(cfg, B, P, N, group_size=64, device="cuda", seed=0, cuda_graphs=not args.no_cuda_graphs)
        launches_of = lambda: native.LAUNCHES["count"]  # noqa: E731
        kernels_of = lambda: native.LAUNCHES["by_kernel"]  # noqa: E731
    setup_s = time.perf_counter() - t0
    dist = torch.distributed if world > 1 else None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    rs = np.random.RandomState(0)
    prompts = [torch.from_numpy(rs.randint(0, cfg.vocab_size, (B, P)).astype(np.int32)).pin_memory() for _ in range(W + K)]
    for i in range(W):
        out = gen.generate(prompts[i])
    launches0 = launches_of()
    dev_ms = prefill_ms = decode_ms = 0.0
    with ClockSampler(local_rank) as clocks:
        barrier()
        t1 = time.perf_counter()
        for i in range(K):
            out = gen.generate(prompts[W + i])  # pinned prompt -> device, program, tokens -> host
            prefill_ms += gen.prefill_ms()
            decode_ms += gen.decode_ms()
        barrier()
        e2e_s = time.perf_counter() - t1
    dev_ms = prefill_ms + decode_ms  # CUDA events recorded by the program around its two phases
    launches = launches_of() - launches0
    times = torch.tensor([dev_ms, e2e_s * 1e3, prefill_ms, decode_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, prefill_ms, decode_ms = (float(t) for t in times)
    if args.impl != "torch":
        native.check_gemm_errors()
    if rank == 0:
        toks = B * N * K
        line = {
            "impl": args.impl, "metric": DECODE_METRIC, "value": toks / (dev_ms / 1e3), "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 activations and KV cache, int4 weights (fp16 scales)",
            "data": "synthetic (uniform random prompt ids, random-init N(0,0.02) weights quantised to int4)",
            "config": {"model": f"{args.model} ({cfg.layers} layers, hidden {cfg.hidden}, {cfg.heads} heads x "
                                f"{cfg.head_dim}, ffn {cfg.ffn}, vocab {cfg.vocab_size})",
                       "global_batch": B, "seq_len": P + N, "prompt_len": P, "new_tokens": N,
                       "parallelism": f"tp{args.gpus}", "group_size": 64,
                       "cuda_graphs": not args.no_cuda_graphs,
                       "torch_weights": ("bf16 copy cached" if args.torch_dense else "int4, de-quantised per call")
                       if args.impl == "torch" else None,
                       "l2": "every decoding step streams all int4 weights and the KV cache (several GB in total), "
                             "beyond the 126 MB L2; no flush needed",
                       "headline": (not args.layers and not args.emulate_tp and args.model == "gptj_6b"
                                    and (B, P, N) == (16, 512, 128)),
                       "emulate_tp": args.emulate_tp or None},
            "clocks": clocks.summary(),
            "e2e": {"value": toks / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": B * P * 4, "d2h_bytes_per_step": B * N * 4},
            "gpu_launches": int(launches), "kernels": kernels_of(),
            "prefill_ms": prefill_ms / K, "decode_ms": decode_ms / K,
            "decode_only_tokens_per_s": B * (N - 1) * K / (decode_ms / 1e3),
            "ms_per_decode_step": decode_ms / K / (N - 1),
            "sample_tokens": [int(t) for t in np.asarray(out)[0, :8]], "setup_seconds": setup_s,
        }
        print(json.dumps(line))
    _shutdown(dist)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="gptj_6b")
    ap.add_argument("--micro-batches", type=int, default=16)
    ap.add_argument("--micro-batch-size", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (diagnostics only; such a run is "
                                                         "labelled and is not the headline configuration)")
    ap.add_argument("--mode", default="train", choices=["train", "decode", "pipeline"],
                    help="train: the training step (default, headline); decode: int4 greedy generation, TP over all GPUs; "
                         "pipeline: pipeline x data parallel training (--stages device slots per replica)")
    ap.add_argument("--tp", type=int, default=0, help="train mode: tensor-parallel width (default min(gpus, 4))")
    ap.add_argument("--stages", type=int, default=4, help="pipeline mode: device slots (GPUs) per replica")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="train mode: shard the residual stream over the tokens inside the TP group")
    ap.add_argument("--no-recompute", action="store_true",
                    help="train / pipeline mode, both arms: keep the activations of every layer instead of running each "
                         "block's forward pass a second time (a micro-batch of 2048 tokens keeps about 6 GB at TP1)")
    ap.add_argument("--prune-recompute", action="store_true",
                    help="train / pipeline mode: the recomputed forward pass of a block leaves out the ops that only lead "
                         "to the block's output (also XL_PRUNE_RECOMPUTE=1); the gradients are bit-identical")
    ap.add_argument("--batch", type=int, default=16, help="decode mode: sequences per batch")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="diagnostics: run ONE rank's shard shapes of a K-way tensor-parallel layout (heads, ffn and "
                         "vocabulary divided by K, no collectives) to separate kernel time from communication")
    ap.add_argument("--torch-dense", action="store_true",
                    help="decode mode, --impl torch: keep a bf16 copy of every weight instead of de-quantising per call")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.mode == "decode":
        return run_decode(args)

    import torch

    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    tp, dp = layout_for(args.gpus)
    if args.tp:
        tp, dp = args.tp, args.gpus // args.tp
    pipeline = args.mode == "pipeline"
    if pipeline:
        if args.impl != "ours":
            raise SystemExit("pipeline mode has no --impl torch arm")
        stages = min(args.stages, args.gpus)
        tp, dp = 1, args.gpus // stages
        if args.model == "gptj_6b":
            args.model = "llama2_7b"
        if args.micro_batches == 16:
            args.micro_batches = 32
    cfg = getattr(DecoderConfig, args.model)(tp=tp, dp=dp)
    if args.layers:
        cfg.layers = args.layers
    if args.emulate_tp:
        _shrink(cfg, args.emulate_tp)
    cfg.sequence_parallel = bool(args.sequence_parallel)
    W = max(args.warmup, 3)
    K = args.steps
    t0 = time.perf_counter()
    if args.impl == "torch":
        # PyTorch + cuBLAS + flash SDPA + NCCL implementation of the same step (the number to beat on this machine)
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        from torch_decoder import TorchTrainer

        class _NoNative:
            LAUNCHES = {"count": 0, "by_kernel": {}}

            @staticmethod
            def check_gemm_errors():
                pass

        native = _NoNative
        tt = TorchTrainer(cfg, micro_batches=args.micro_batches, recompute=not args.no_recompute)

        class _Adapter:
            tokens_per_step = tt.tokens_per_step

            class session:
                h2d_bytes = 0
                d2h_bytes = 0

            def synthetic_tokens(self, seed=0):
                g = torch.Generator().manual_seed(seed + rank // max(tp, 1))
                return torch.randint(0, cfg.vocab_size, (args.micro_batches, 1, 1, cfg.seq_len + 1), generator=g,
                                     dtype=torch.int32).pin_memory()

            def step(self, t):
                _Adapter.session.h2d_bytes += t.numel() * 4
                _Adapter.session.d2h_bytes += 4
                return tt.step(t)

            def step_device(self, t):
                return tt.step_device(t)

        trainer = _Adapter()
    elif pipeline:
        from popxl_addons_b200.models.pipeline_trainer import PipelineTrainer
        from popxl_addons_b200.ops import native

        trainer = PipelineTrainer(cfg, stages=stages, micro_batches=args.micro_batches,
                                  micro_batch_size=args.micro_batch_size, device="cuda", seed=0, lr=1e-4,
                                  recompute=not args.no_recompute,
                                  prune_recompute=True if args.prune_recompute else None)
    else:
        trainer = DecoderTrainer(cfg, micro_batches=args.micro_batches, micro_batch_size=args.micro_batch_size,
                                 device="cuda", seed=0, lr=1e-4, recompute=not args.no_recompute,
                                 prune_recompute=True if args.prune_recompute else None)
        from popxl_addons_b200.ops import native
    setup_s = time.perf_counter() - t0

    dist = torch.distributed if world > 1 else None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    host_tokens = [trainer.synthetic_tokens(seed=i) for i in range(W + K)]
    dev_tokens = [t.cuda(non_blocking=True) for t in host_tokens]
    losses = []
    for i in range(W):
        losses.append(trainer.step(host_tokens[i]))
    if pipeline:
        # only the last slot of a replica sees the loss: share it for the report
        losses = [l if l is not None else float("nan") for l in losses]

    # ---- device-timed region: K steps, inputs resident, CUDA events, max over ranks ----------------------------------
    launches0 = native.LAUNCHES["count"]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        start.record()
        last = None
        for i in range(K):
            last = trainer.step_device(dev_tokens[W + i])
        end.record()
        barrier()
    dev_ms = start.elapsed_time(end)
    launches = native.LAUNCHES["count"] - launches0
    native.check_gemm_errors()

    # ---- end to end through the public API: H2D of the tokens from pinned memory + D2H of the losses, every step ---------
    h2d0, d2h0 = trainer.session.h2d_bytes, trainer.session.d2h_bytes
    barrier()
    t1 = time.perf_counter()
    for i in range(K):
        losses.append(trainer.step(host_tokens[W + i]))
    barrier()
    e2e_s = time.perf_counter() - t1
    if pipeline and dist is not None:
        box = [losses]
        dist.broadcast_object_list(box, src=stages - 1)  # the last slot of replica 0 computes the loss
        losses = box[0]
    h2d = (trainer.session.h2d_bytes - h2d0) // K
    d2h = (trainer.session.d2h_bytes - d2h0) // K

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens = trainer.tokens_per_step
    value = tokens * K / (dev_ms / 1e3)
    e2e_value = tokens * K / (e2e_ms / 1e3)
    if rank == 0:
        flops_per_token = 6 * cfg.param_count() + 6 * cfg.layers * cfg.seq_len * cfg.heads * cfg.head_dim
        line = {
            "impl": args.impl, "metric": PIPELINE_METRIC if pipeline else METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": f"{args.model} ({cfg.layers} layers, hidden {cfg.hidden}, {cfg.heads} heads x "
                                f"{cfg.head_dim}, ffn {cfg.ffn}, vocab {cfg.vocab_size})",
                       "global_batch": args.micro_batches * args.micro_batch_size * dp, "seq_len": cfg.seq_len,
                       "parallelism": (f"pp{stages}xdp{dp}" if pipeline else f"tp{tp}xdp{dp}"), "micro_batches": args.micro_batches, "micro_batch_size": args.micro_batch_size,
                       "optimizer": "AdamW, fp32 master weights + fp32 moments" +
                                    (", state sharded over dp (RTS)" if dp > 1 else ""),
                       "recompute": "none (activations kept)" if args.no_recompute else "per layer" + (
                           ", second forward pass reduced to what the backward pass reads"
                           if args.impl == "ours" and trainer.prune_recompute else ""), "l2": "each step streams >100 GB of weights, optimizer state and "
                                                       "activations, far beyond the 126 MB L2; no flush needed",
                       "emulate_tp": args.emulate_tp or None, "sequence_parallel": bool(args.sequence_parallel),
                       "headline": (not args.layers and not args.emulate_tp and args.model == "gptj_6b" and not pipeline
                                    and not args.tp
                                    and args.micro_batch_size == 1 and args.micro_batches == 16)},
            "clocks": clocks.summary(),
            "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / K, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches),
            "kernels": native.LAUNCHES["by_kernel"],
            "model_tflops_per_gpu": flops_per_token * value / args.gpus / 1e12,
            "loss_first_last": [losses[0], losses[-1]], "setup_seconds": setup_s, "mode": args.mode,
        }
        print(json.dumps(line))
    _shutdown(dist)
    return 0


if __name__ == "__main__":
    sys.exit(main())
