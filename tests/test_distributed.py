"""One process per replica (the production layout) against the in-process replica simulation: CPU ranks over gloo here,
GPU ranks over NCCL + the fused NVLink kernels on a multi-GPU box. Also host-side failure detection."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(nproc, *worker_args, timeout=600, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "dist_worker.py"),
           *worker_args]
    e = dict(os.environ)
    e.update(env or {})
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert lines, f"worker produced no result\nstdout:\n{res.stdout[-3000:]}\nstderr:\n{res.stderr[-3000:]}"
    return json.loads(lines[-1])


def simulated(tp, dp, dtype, steps=3, big=False, fused=True, sp=False):
    from popxl_addons_b200.models import decoder as dec
    from popxl_addons_b200.models.gptj import GPTJConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer
    sys.path.insert(0, HERE)
    from dist_worker import global_tokens

    dec._SEED[0] = 0
    cfg = (GPTJConfig.tiny(dtype=dtype, tp=tp, dp=dp, **({"seq_len": 512} if big == 2 else {})) if big
           else dec.DecoderConfig.tiny("gptj", dtype=dtype, tp=tp, dp=dp))
    cfg.sequence_parallel = bool(sp)
    t = DecoderTrainer(cfg, micro_batches=2, device="cpu", lr=1e-2 if big != 2 else 2e-3, fused_collectives=fused)
    return [t.step(global_tokens(cfg, 2, seed=s)) for s in range(steps)]


def test_fused_ops_equal_unfused_composition_in_simulation():
    a = simulated(2, 2, "float32", fused=False)
    b = simulated(2, 2, "float32", fused=True)
    np.testing.assert_allclose(a, b, rtol=1e-6)


@pytest.mark.parametrize("tp,dp", [(1, 2), (2, 1)])
def test_cpu_ranks_match_simulation(tp, dp):
    ref = simulated(tp, dp, "float32")
    got = launch(2, "--device", "cpu", "--tp", str(tp), "--dp", str(dp), "--dtype", "float32")
    np.testing.assert_allclose(got["losses"], ref, rtol=2e-4)


def test_cpu_ranks_with_pruned_recomputation_match_simulation():
    """Every rank leaves the same all-reduce out of its recomputed forward pass, so the ranks stay in step."""
    ref = simulated(2, 1, "float32")
    got = launch(2, "--device", "cpu", "--tp", "2", "--dp", "1", "--dtype", "float32", env={"XL_PRUNE_RECOMPUTE": "1"})
    np.testing.assert_allclose(got["losses"], ref, rtol=2e-4)


def test_cpu_ranks_with_asynchronous_all_reduces_match_simulation():
    """All-reduces issued asynchronously and joined before their first reader, in graphs reordered so that the
    weight-gradient GEMMs run in between (also together with the pruned second forward pass)."""
    ref = simulated(2, 1, "float32")
    for extra in ({}, {"XL_PRUNE_RECOMPUTE": "1"}):
        got = launch(2, "--device", "cpu", "--tp", "2", "--dp", "1", "--dtype", "float32",
                     env={"XL_ASYNC_COLLECTIVES": "1", "XL_FUSE_GEMM_AR": "0", **extra})
        np.testing.assert_allclose(got["losses"], ref, rtol=2e-4)


def test_cpu_rank_collectives():
    assert launch(2, "--mode", "collectives", "--device", "cpu")["ok"]


def test_rank_loss_is_detected_on_the_host():
    res = launch(2, "--mode", "fail", timeout=120)
    assert res["detected"] and res["missing"] == [1] and res["step"] == 2


def test_supervisor_restarts_from_the_latest_checkpoint(tmp_path):
    """Rank 1 fails on the host after step 3 of the first attempt: rank 0 learns it from the heartbeat and leaves, the
    supervisor starts the job again, both ranks resume from the checkpoint of step 2 and finish. The result equals the
    uninterrupted run bit for bit (CPU ranks over gloo)."""
    from popxl_addons_b200.parallel.elastic import Supervisor, latest_checkpoint

    worker = os.path.join(HERE, "dist_worker.py")
    results = {}
    for name, inject in (("plain", "0"), ("interrupted", "1")):
        root = tmp_path / name
        root.mkdir()
        sup = Supervisor([worker, "--mode", "elastic", "--steps", "6", "--ckpt", str(root)], nproc=2, max_restarts=2,
                         env={"XL_TEST_INJECT_FAILURE": inject}, grace_s=30.0, log=lambda m: None)
        assert sup.run() == 0
        with open(root / "result.json") as f:
            results[name] = (json.load(f), sup.attempts)
        assert latest_checkpoint(str(root)).endswith("step6")
    plain, attempts = results["plain"]
    assert attempts == [[0, 0]] and plain["attempt"] == 0 and plain["resumed_from"] == 0 and plain["steps"] == 6
    got, attempts = results["interrupted"]
    assert len(attempts) == 2 and attempts[0] == [3, 7] and attempts[1] == [0, 0]
    assert got["attempt"] == 1 and got["resumed_from"] == 2 and got["steps"] == 6
    assert got["w"] == plain["w"] and got["w_sum"] == plain["w_sum"]
    assert [got["losses"][str(s)] for s in range(2, 6)] == [plain["losses"][str(s)] for s in range(2, 6)]
    # a directory without session_info.json (a checkpoint that was being written) is not picked up
    (tmp_path / "plain" / "step8" / "model").mkdir(parents=True)
    assert latest_checkpoint(str(tmp_path / "plain")).endswith("step6")
    assert latest_checkpoint(str(tmp_path / "nothing")) is None


def _need_gpus(n):
    import torch

    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if have < n:
        pytest.skip(f"needs {n} CUDA devices, {have} present")


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("tp,dp", [(1, 2), (2, 1), (2, 2), (4, 1), (4, 2)])
def test_gpu_ranks_fused_collectives(tp, dp):
    """bf16 on tp x dp GPUs (2, 4 or 8): the fused NVLink kernels must have run and two optimizer steps must track the
    fp32-accumulating CPU simulation of the same program."""
    _need_gpus(tp * dp)
    big = 2 if tp > 1 else 1  # 512 tokens per micro-batch: whole 128-row blocks for every rank of the TP group
    ref = simulated(tp, dp, "bfloat16", big=big)
    got = launch(tp * dp, "--device", "cuda", "--tp", str(tp), "--dp", str(dp), "--dtype", "bfloat16", "--big", str(big),
                 timeout=600)
    np.testing.assert_allclose(got["losses"], ref, rtol=3e-2)
    kernels = got["kernels"]
    assert "gemm_tcgen05" in kernels or "gemm2cta_tcgen05" in kernels
    if dp > 1:
        # the sharded optimizer step ran as the one-launch-per-bucket kernel (or the per-tensor one) over peer memory
        assert kernels.get("rts_adam_bucket", 0) + kernels.get("rts_adam", 0) > 0, kernels
    if tp > 1:
        assert got["fused_pairs"] > 0
        assert kernels.get("gemm_ar_pull_tcgen05", 0) > 0, kernels  # the TP all-reduce ran inside the GEMM kernel
        assert kernels.get("ce_shard_stats", 0) > 0 and kernels.get("ce_shard_grad_loss", 0) > 0, kernels
        assert not got.get("fallbacks"), got.get("fallbacks")


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("tp", [2, 4])
def test_gpu_ranks_sequence_parallel(tp):
    """Sequence parallelism on GPUs: the residual stream sharded over the tokens of the TP group, reduce-scatter by
    pulling inside the row-parallel GEMMs, all-gather by multicast before the column-parallel ones; must track the CPU
    simulation of the same program."""
    _need_gpus(tp)
    ref = simulated(tp, 1, "bfloat16", big=2, sp=True)
    got = launch(tp, "--device", "cuda", "--tp", str(tp), "--dp", "1", "--dtype", "bfloat16", "--big", "2", "--sp", "1",
                 timeout=600)
    np.testing.assert_allclose(got["losses"], ref, rtol=3e-2)
    kernels = got["kernels"]
    assert kernels.get("gemm_rs_pull_tcgen05", 0) > 0 and kernels.get("symm_all_gather_mc", 0) > 0, kernels
    assert not got.get("fallbacks") or all(k.startswith("fused:") for k in got["fallbacks"]), got.get("fallbacks")


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4])
def test_gpu_rts_bucket_optimizer_with_and_without_clipping(nproc):
    """One launch per bucket: reduce-scatter + AdamW + all-gather fused, and the clipped form (reduce + sum of squares,
    global norm, update from the reduced gradients), against numpy AdamW on the averaged gradients."""
    _need_gpus(nproc)
    res = launch(nproc, "--mode", "rtsclip", "--device", "cuda", timeout=300)
    assert res["errors"]["fused"] < 1e-2 and res["errors"]["clip"] < 1e-2, res  # bf16 weights: 2^-8 relative
    assert res["kernels"].get("rts_adam_bucket", 0) == 2 and res["kernels"].get("rts_reduce_bucket", 0) == 1, res


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_rank_collectives():
    assert launch(2, "--mode", "collectives", "--device", "cuda")["ok"]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("nproc,m,n,k", [(2, 1024, 1024, 1024), (2, 512, 2304, 384), (4, 1024, 1024, 1024),
                                         (4, 2048, 4096, 1024)])
def test_gpu_gemm_reduce_scatter_and_all_gather_gemm(nproc, m, n, k):
    """The tcgen05 GEMM fused with its collective, against NCCL + fp32 matmul on the same data, on 2 and 4 ranks and
    more than one shape: the reduce-scatter epilogue (`red.add` into the owner's shard), the all-gather prologue (copy
    CTAs pulling peer row blocks), the pushing all-reduce (`multimem.red`) and the pulling all-reduce
    (`multimem.ld_reduce` / `multimem.st` by the owner of the rows; one and two operand pairs, both weight layouts,
    many launches back to back)."""
    _need_gpus(nproc)
    res = launch(nproc, "--mode", "fusedgemm", "--gemm-m", str(m), "--gemm-n", str(n), "--gemm-k", str(k), timeout=300,
                 env={"XL_COLLECTIVE_TIMEOUT_S": "120"})
    assert res["errors"] is None
    assert res["rs_err"] < 2e-2 and res["ag_a_err"] < 2e-2 and res["ag_b_err"] < 2e-2 and res["ar_err"] < 2e-2
    assert res["ar_pull_err"] < 2e-2 and res["ar_pull2_err"] < 2e-2 and res["ar_pull2_t_err"] < 2e-2, res
    assert res["ar_pull2_repeat_err"] < 2e-2, res
    assert res["rs_pull2_err"] < 2e-2 and res["ag_mc_ok"] and res["ag_mc_repeat_ok"], res
    assert res["ag_a_gathered_ok"] and res["ag_b_gathered_ok"]
    assert res["ar_ln_err"] < 0.1  # bf16 rounding of the summed update (magnitudes ~ 4)


@pytest.mark.parametrize("nproc", [2, 4])
def test_pipeline_stages_on_separate_processes(nproc):
    """A replica spanning two processes (one per device slot, stage boundaries as send/recv) must produce the gradients
    of the same program run sequentially; with 4 processes two such replicas average their gradients."""
    from popxl_addons_b200 import xl as popxl
    import popxl_addons_b200 as addons
    from popxl_addons_b200.layers import Linear

    steps, R = 6, nproc // 2
    np.random.seed(42)
    data = np.random.normal(0, 1, (steps, R, 1, 4)).astype(np.float32)
    grads = []
    for r in range(R):
        np.random.seed(42)
        np.random.normal(0, 1, (steps, R, 1, 4))  # same generator position as in the workers
        ir = popxl.Ir()
        with ir.main_graph:
            _, x_stream, x = addons.host_load(data[0, 0], popxl.float32, "x")
            fargs, lin = Linear(4).create_graph(x)
            dargs, dlin = addons.autodiff_with_accumulation(lin, [lin.args.weight])
            w, dw = fargs.init(), dargs.init()
            info = lin.bind(w).call_with_info(x)
            y, *_ = info.outputs
            y = y * 2.0 + 1
            dlin.bind(dw).call(y, args=dlin.grad_graph_info.inputs_dict(info))
        with popxl.Session(ir, "cpu") as s:
            for n in range(steps):
                s.run({x_stream: data[n, r]})
        grads.append(s.get_tensor_data(dw.accum.weight).copy())
    want = np.mean(grads, axis=0).reshape(-1)
    res = launch(nproc, "--mode", "pipeline", "--slots", "2", timeout=240)
    for info in res["ranks"]:
        assert info["owned"] == ({"w": True, "dw": True, "scale": False} if info["slot"] == 0 else
                                 {"w": False, "dw": False, "scale": True})
        if info["slot"] == 0:
            np.testing.assert_allclose(info["grad"], want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("nproc", [2, 4])
def test_pipeline_trainer_on_separate_processes_matches_simulation(nproc, tmp_path):
    """Llama-shaped model, 2 device slots per replica, 1 or 2 data-parallel replicas: the losses of three optimizer steps
    must match the same trainer run in one process (all slots and replicas simulated in-process)."""
    from popxl_addons_b200.models import decoder as dec
    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.pipeline_trainer import PipelineTrainer

    dp = nproc // 2
    cfg = DecoderConfig.tiny("llama", layers=4, dtype="float32", tp=1, dp=dp)
    dec._SEED[0] = 0
    tr = PipelineTrainer(cfg, stages=2, micro_batches=6, device="cpu", lr=1e-2)
    want = []
    for step in range(3):
        g = torch.Generator().manual_seed(step)
        tok = torch.randint(0, cfg.vocab_size, (6, dp, 1, cfg.seq_len + 1), generator=g, dtype=torch.int32)
        out = tr.session.run({tr.inputs.tokens: tok, tr.inputs.labels: tok})[tr.outputs.loss]
        want.append(np.asarray(out).reshape(6, dp).mean(axis=0))  # per replica
    ckpt = str(tmp_path / "ckpt")
    res = launch(nproc, "--mode", "pp_train", "--slots", "2", "--dtype", "float32", "--ckpt", ckpt, timeout=400)
    # checkpoint: one directory, every variable exactly once (written by the slot that owns it), restored bit-exactly
    files = {os.path.basename(p)[:-4] for p in os.listdir(os.path.join(ckpt, "model"))}
    assert len(files) == res["n_state"] and os.path.exists(os.path.join(ckpt, "session_info.json"))
    assert sum(i["n_owned"] for i in res["ranks"][:2]) == res["n_state"]
    for info in res["ranks"]:
        assert info["ckpt_ok"] is True
        replica, slot = info["rank"] // 2, info["rank"] % 2
        if slot == 1:
            np.testing.assert_allclose(info["losses"], [w[replica] for w in want], rtol=1e-4)
        else:
            assert info["losses"] == [None] * 3


def test_sequence_parallel_equals_plain_tensor_parallel():
    """Residual stream sharded over the tokens inside the TP group (reduce-scatter / all-gather instead of all-reduce):
    same losses as the plain TP program, in the in-process simulation and with one process per replica (gloo)."""
    import dataclasses

    from popxl_addons_b200.models import decoder as dec
    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer
    sys.path.insert(0, HERE)
    from dist_worker import global_tokens

    results = {}
    for family in ("gptj", "llama", "gpt2"):
        cfg = DecoderConfig.tiny(family, dtype="float32", tp=2, dp=1)
        for sp in (False, True):
            dec._SEED[0] = 0
            tr = DecoderTrainer(dataclasses.replace(cfg, sequence_parallel=sp), micro_batches=2, device="cpu", lr=1e-2)
            results[family, sp] = [tr.step(global_tokens(cfg, 2, seed=s)) for s in range(3)]
        np.testing.assert_allclose(results[family, True], results[family, False], rtol=1e-5)
    got = launch(2, "--device", "cpu", "--tp", "2", "--dp", "1", "--dtype", "float32", "--sp", "1")
    np.testing.assert_allclose(got["losses"], results["gptj", False], rtol=1e-4)


def test_supervisor_policies(tmp_path):
    """Restart budget, workers that outlive a failed peer (stopped by their own pids after the grace period) and
    workers that die from a signal, with plain scripts in place of training processes."""
    from popxl_addons_b200.parallel.elastic import Supervisor

    script = tmp_path / "worker.py"
    script.write_text(
        "import os, signal, sys, time\n"
        "rank, attempt, mode = int(os.environ['RANK']), int(os.environ['XL_RESTART_COUNT']), sys.argv[1]\n"
        "assert os.environ['WORLD_SIZE'] == '2' and os.environ['MASTER_ADDR'] == '127.0.0.1'\n"
        "if mode == 'flaky' and attempt < 2 and rank == 1: sys.exit(5)\n"
        "if mode == 'always' and rank == 0: sys.exit(9)\n"
        "if mode == 'hang' and attempt == 0:\n"
        "    if rank == 0: sys.exit(4)\n"
        "    time.sleep(600)\n"
        "if mode == 'signal' and attempt == 0 and rank == 1: os.kill(os.getpid(), signal.SIGKILL)\n"
        "open(os.path.join(os.path.dirname(__file__), f'done_{mode}_{rank}'), 'w').write(str(attempt))\n")
    quiet = dict(log=lambda m: None, poll_s=0.02)
    flaky = Supervisor([str(script), "flaky"], nproc=2, max_restarts=3, grace_s=5.0, **quiet)
    assert flaky.run() == 0 and len(flaky.attempts) == 3 and flaky.attempts[-1] == [0, 0]
    assert (tmp_path / "done_flaky_1").read_text() == "2"
    always = Supervisor([str(script), "always"], nproc=2, max_restarts=1, grace_s=5.0, **quiet)
    assert always.run() == 9 and len(always.attempts) == 2  # the budget is spent, the failing status is returned
    hang = Supervisor([str(script), "hang"], nproc=2, max_restarts=1, grace_s=0.3, **quiet)
    assert hang.run() == 0 and hang.attempts[0][0] == 4 and hang.attempts[0][1] < 0  # the sleeper was signalled
    sig = Supervisor([str(script), "signal"], nproc=2, max_restarts=1, grace_s=5.0, **quiet)
    assert sig.run() == 0 and sig.attempts[0][1] == -9 and sig.attempts[1] == [0, 0]
    none = Supervisor([str(script), "always"], nproc=2, max_restarts=0, grace_s=1.0, **quiet)
    assert none.run() == 9 and len(none.attempts) == 1
