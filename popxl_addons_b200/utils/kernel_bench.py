"""Per-kernel timing against the roofline: `python -m popxl_addons_b200.utils.kernel_bench [--peaks MEASURED_PEAKS.json]`.

Times every hot kernel on shapes of the GPT-J-6B configuration with CUDA events (3 warm-up + 10 timed launches, an L2
flush between launches) and reports achieved TFLOP/s or GB/s as a fraction of the measured peaks, next to the library
kernel (cuBLAS / torch) on the same shape for reference.
"""
import argparse
import json
import os

import torch


def _flush():
    if not hasattr(_flush, "buf"):
        _flush.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.buf.zero_()


def time_ms(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        _flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def graph_time_ms(fn, reps=40, iters=5):
    """Device time of one launch of a short kernel: `reps` back-to-back launches captured in a CUDA graph and replayed
    (no host launch path in the timed region), median over `iters` replays, divided by `reps`. Caches stay warm, which
    is what a decode step replayed from a graph sees for its small activations (the weights still stream from HBM when
    they exceed L2)."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / reps)
    times.sort()
    return times[len(times) // 2]


def attention_trace(nat, H, S=2048, D=256):
    """Where an iteration (one key block) of the attention kernels goes: SM clock stamps taken by the MMA-issuing thread
    and by the first softmax / element-wise warp of CTA (0, 0, 0), which owns the last query block."""
    import math

    hd = H * D
    torch.manual_seed(0)
    qkv = (torch.randn(S, 3 * hd, device="cuda") * 0.5).bfloat16()
    do = (torch.randn(S, hd, device="cuda") * 0.5).bfloat16()
    scale = 1 / math.sqrt(D)

    def stamps(run):
        trace = torch.zeros(2 * 64 * 8, dtype=torch.int64, device="cuda")
        for _ in range(3):
            run(None)
        run(trace)
        torch.cuda.synchronize()
        t = trace.view(2, 64, 8).cpu()
        return t, int(t[t > 0].min()), int((t[0, :, 0] > 0).sum())

    def show(t, t0, n, role, cols, label):
        print(label)
        for j in list(range(min(n, 4))) + list(range(max(4, n - 2), n)):
            print("   block %2d" % j, [int(t[role, j, k]) - t0 if t[role, j, k] > 0 else -1 for k in cols])

    t, t0, n = stamps(lambda tr: nat.flash_attention_fwd(qkv, 0, hd, 2 * hd, 1, S, H, D, scale, True, trace=tr))
    print(f"forward, {H} heads: {n} key blocks of 64 in CTA 0")
    show(t, t0, n, 0, (0, 1, 2, 3, 4), "  MMA thread: iteration start | scores of block j+1 issued | V_j there | P_j there | P_j V_j issued")
    show(t, t0, n, 1, (0, 1, 2, 3, 4, 5), "  softmax warp: enter | S_j there | loaded | exponentials done | previous PV done | P_j written")
    m = t[0, :, 0].double()
    print("  clocks per iteration:", round(float((m[n - 1] - m[1]) / max(1, n - 2))))
    out, lse = nat.flash_attention_fwd(qkv, 0, hd, 2 * hd, 1, S, H, D, scale, True)
    dqkv = torch.empty_like(qkv)
    t, t0, n = stamps(lambda tr: nat.flash_attention_bwd_dq(qkv, out, do, lse, dqkv, 1, S, H, D, scale, True, trace=tr))
    print(f"backward (dQ pass), {H} heads: {n} key blocks of 32 in CTA 0")
    show(t, t0, n, 0, (0, 1, 2, 3), "  MMA thread: iteration start | S and dP of block j+1 issued | dS_j there | dQ += dS_j K_j issued")
    show(t, t0, n, 1, (0, 1, 2, 3, 5, 6, 4), "  element-wise warp: enter | S, dP there | loaded | P, dS computed | dS buffer free | dS in shared memory | P, dS in global memory")
    m = t[0, :, 0].double()
    print("  clocks per iteration:", round(float((m[n - 1] - m[1]) / max(1, n - 2))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--peaks", default=os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json"))
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default=None, help="run only the rows whose name contains this text (profiler captures)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--attention-trace", type=int, default=0, metavar="HEADS",
                    help="print the clock stamps that the first CTA of the attention kernels records (forward and "
                         "backward, sequence 2048, head dimension 256, this many heads) and exit")
    args = ap.parse_args()
    want = (lambda name: args.only is None or args.only in name)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    src = "fallback"
    if os.path.exists(args.peaks):
        peaks.update(json.load(open(args.peaks)))
        src = "measured"
    from popxl_addons_b200.ops import native as nat

    if args.attention_trace:
        attention_trace(nat, args.attention_trace)
        return
    rows = []
    bf = torch.bfloat16

    def gemm_row(name, M, N, K, a_t=False, b_t=False, batch=1, mean_into_fp32=False):
        """Device time of one launch, from a replayed graph of back-to-back launches that walk round-robin through
        enough operand sets to exceed L2 (so every launch streams its operands from HBM, as inside a training step, and
        the host launch path of a short kernel is not in the number). Both tcgen05 kernels and cuBLAS on every shape."""
        if not want(name):
            return
        per_set = 2 * batch * (M * K + K * N + M * N)
        n_sets = max(1, min(8, -(-300_000_000 // per_set)))
        sets = []
        for _ in range(n_sets):
            a = torch.randn((batch, K, M) if a_t else (batch, M, K), device="cuda", dtype=bf)
            b = torch.randn((batch, N, K) if b_t else (batch, K, N), device="cuda", dtype=bf)
            av = a.transpose(-1, -2) if a_t else a
            bv = b.transpose(-1, -2) if b_t else b
            if batch == 1:
                av, bv = av[0], bv[0]
            sets.append((av, bv, torch.zeros((batch, M, N) if batch > 1 else (M, N), device="cuda",
                                             dtype=torch.float32 if mean_into_fp32 else bf)))
        reps = max(n_sets, 24 // n_sets * n_sets)

        def rotating(fn):
            state = {"i": 0}

            def call():
                av, bv, out = sets[state["i"] % n_sets]
                state["i"] += 1
                return fn(av, bv, out)

            return call

        fl = 2.0 * M * N * K * batch
        if mean_into_fp32:
            # weight gradient folded into an fp32 accumulator (running mean over micro-batches) by the GEMM's epilogue;
            # the library form is a product in 16 bits followed by an in-place update of the accumulator
            step = torch.full((1,), 3.0, device="cuda")
            tmp = torch.empty((M, N), device="cuda", dtype=bf)

            def lib_fn(av, bv, out):
                torch.matmul(av, bv, out=tmp)
                return out.mul_(0.75).add_(tmp, alpha=0.25)

            lib = graph_time_ms(rotating(lib_fn), reps=reps)
            ours_fn = lambda av, bv, out: nat.gemm(av, bv, out=out, accumulate=2, step=step)  # noqa: E731
        else:
            lib = graph_time_ms(rotating(lambda av, bv, out: torch.matmul(av, bv, out=out)), reps=reps)
            ours_fn = lambda av, bv, out: nat.gemm(av, bv, out=out)  # noqa: E731
        saved, saved_tile = nat._GEMM_CTA_PAIRS, nat._GEMM_PAIR_TILE_N[0]
        try:
            # CTA pairs with the tile width picked per shape (the default), with each width forced, and the single-CTA kernel
            for pairs, tile_n, tag in ((True, 0, " [CTA pairs]"), (True, 256, " [CTA pairs, 256-wide tiles]"),
                                       (True, 128, " [CTA pairs, 128-wide tiles]"), (False, 0, " [single CTA]")):
                nat._GEMM_CTA_PAIRS, nat._GEMM_PAIR_TILE_N[0] = pairs, tile_n
                if pairs and N <= 128:
                    continue
                ours = graph_time_ms(rotating(ours_fn), reps=reps)
                rows.append(dict(kernel=name + tag,
                                 shape=f"{batch}x{M}x{N}x{K}", ms=ours, tflops=fl / ours / 1e9,
                                 frac_of_peak=fl / ours / 1e9 / peaks["bf16_tflops"], lib_ms=lib,
                                 lib_tflops=fl / lib / 1e9, vs_lib=lib / ours))
        finally:
            nat._GEMM_CTA_PAIRS, nat._GEMM_PAIR_TILE_N[0] = saved, saved_tile

    gemm_row("gemm fwd qkv", 2048, 12288, 4096)
    gemm_row("gemm fwd fc_in", 2048, 16384, 4096)
    gemm_row("gemm fwd fc_out", 2048, 4096, 16384)
    gemm_row("gemm dgrad fc_in (B K-major)", 2048, 4096, 16384, b_t=True)
    gemm_row("gemm wgrad fc_in (A,B MN-major)", 4096, 16384, 2048, a_t=True)
    gemm_row("gemm wgrad fc_in into fp32 mean (A,B MN-major)", 4096, 16384, 2048, a_t=True, mean_into_fp32=True)
    gemm_row("gemm lm_head", 2048, 50400, 4096)
    gemm_row("gemm wgrad lm_head into fp32 mean (A,B MN-major)", 4096, 50400, 2048, a_t=True, mean_into_fp32=True)
    gemm_row("gemm attn scores", 2048, 2048, 256, b_t=True, batch=16)
    gemm_row("gemm attn pv", 2048, 256, 2048, batch=16)
    gemm_row("gemm square 8192", 8192, 8192, 8192)
    # one rank's shapes at TP4: 192 to 256 tiles of 128 x 256 on 148 SMs (the second wave is partly empty)
    gemm_row("gemm tp4 fwd qkv", 2048, 3072, 4096)
    gemm_row("gemm tp4 fwd out", 2048, 4096, 1024)
    gemm_row("gemm tp4 fwd fc_in", 2048, 4096, 4096)
    gemm_row("gemm tp4 wgrad fc_in (A,B MN-major)", 4096, 4096, 2048, a_t=True)
    gemm_row("gemm tp4 dgrad out (B K-major)", 2048, 1024, 4096, b_t=True)
    gemm_row("gemm tp4 wgrad out (A,B MN-major)", 1024, 4096, 2048, a_t=True)
    gemm_row("gemm tp4 fwd qkv|fc_in", 2048, 7168, 4096)
    gemm_row("gemm tp4 dgrad qkv (B K-major)", 2048, 4096, 3072, b_t=True)
    gemm_row("gemm tp4 wgrad qkv (A,B MN-major)", 4096, 3072, 2048, a_t=True)

    def attention_row(name, S, H, D):
        """Causal attention forward of one GPT-J micro-batch: the default path (scores GEMM with causal tile skipping,
        fused softmax, PV GEMM) and, with XL_FLASH_ATTENTION=1, the single-kernel forward on the same packed qkv."""
        if not want(name):
            return
        hd = H * D
        qkv = (torch.randn(S, 3 * hd, device="cuda") * 0.5).to(bf)
        sin = torch.zeros(1, S, 1, device="cuda", dtype=bf)
        scale = D ** -0.5
        fl = 2.0 * 2 * S * S * D * H / 2  # two products, half of each masked
        saved, nat._FLASH_ATTENTION = nat._FLASH_ATTENTION, "0"
        try:
            default = graph_time_ms(lambda: nat.attention_qkv_cuda(qkv, sin, sin, S, H, D, 0, True, scale, True), reps=8)
        except Exception:
            raise
        finally:
            nat._FLASH_ATTENTION = saved
        rows.append(dict(kernel=name + " (GEMM + softmax + GEMM)", shape=f"{H}x{S}x{S}x{D}", ms=default,
                         tflops=fl / default / 1e9, frac_of_peak=fl / default / 1e9 / peaks["bf16_tflops"],
                         lib_ms=default, lib_tflops=fl / default / 1e9, vs_lib=1.0, lib_name="GEMM path"))
        one = graph_time_ms(lambda: nat.flash_attention_fwd(qkv, 0, hd, 2 * hd, 1, S, H, D, scale, True), reps=8)
        rows.append(dict(kernel=name + " (single kernel)", shape=f"{H}x{S}x{S}x{D}", ms=one, tflops=fl / one / 1e9,
                         frac_of_peak=fl / one / 1e9 / peaks["bf16_tflops"], lib_ms=default,
                         lib_tflops=fl / default / 1e9, vs_lib=default / one, lib_name="GEMM path"))
        if nat._attention_split("fwd", nat._attn_plan, 1, S, H, D, True, qkv.device)[0] > 0:
            # few heads: the row above divided the keys of a query block over several CTAs; the same kernel without
            saved_split, saved_plans = nat._ATTN_SPLIT, dict(nat._ATTN_PLANS)
            nat._ATTN_SPLIT = False
            nat._ATTN_PLANS.clear()
            try:
                whole = graph_time_ms(lambda: nat.flash_attention_fwd(qkv, 0, hd, 2 * hd, 1, S, H, D, scale, True), reps=8)
            finally:
                nat._ATTN_SPLIT = saved_split
                nat._ATTN_PLANS.clear()
                nat._ATTN_PLANS.update(saved_plans)
            rows.append(dict(kernel=name + " (single kernel, one CTA per query block)", shape=f"{H}x{S}x{S}x{D}", ms=whole,
                             tflops=fl / whole / 1e9, frac_of_peak=fl / whole / 1e9 / peaks["bf16_tflops"], lib_ms=default,
                             lib_tflops=fl / default / 1e9, vs_lib=default / whole, lib_name="GEMM path"))
        # fwd + bwd of the op as the training step runs it (forward as dispatched by default, backward GEMM-based)
        do = torch.randn(S, hd, device="cuda", dtype=bf)

        kw = dict(seq_len=S, n_heads=H, head_dim=D, rotary_dim=0, causal=True, scale=scale)

        def fwd_bwd():
            out, rot, lse = nat.attention_qkv_cuda(qkv, sin, sin, inplace=False, **kw)
            return nat.attention_qkv_grad_cuda(rot, lse, do, sin, sin, out, **kw)

        # 7 products of 2*S*S*D/2 FLOPs per head: 2 forward, 5 backward (scores and dP recomputed / formed once)
        for fused_bwd in (False, True):
            saved_bwd, nat._FLASH_ATTENTION_BWD = nat._FLASH_ATTENTION_BWD, fused_bwd
            try:
                both = graph_time_ms(fwd_bwd, reps=4)
            finally:
                nat._FLASH_ATTENTION_BWD = saved_bwd
            tag = "backward with scores on chip" if fused_bwd else "backward from GEMMs + softmax kernels"
            rows.append(dict(kernel=name.replace("fwd", "fwd+bwd") + f" ({tag})", shape=f"{H}x{S}x{S}x{D}", ms=both,
                             tflops=3.5 * fl / both / 1e9, frac_of_peak=3.5 * fl / both / 1e9 / peaks["bf16_tflops"],
                             lib_ms=both, lib_tflops=3.5 * fl / both / 1e9, vs_lib=1.0, lib_name="itself"))
        # PyTorch's fused scaled-dot-product attention on the same problem (forward + backward), for reference
        q4, k4, v4 = (qkv[:, i * hd:(i + 1) * hd].reshape(1, S, H, D).transpose(1, 2).detach().clone().requires_grad_(True)
                      for i in range(3))
        do4 = do.reshape(1, S, H, D).transpose(1, 2)

        def sdpa():
            o4 = torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, is_causal=True, scale=scale)
            return torch.autograd.grad(o4, (q4, k4, v4), do4)

        try:
            lib = graph_time_ms(sdpa, reps=4)
            rows.append(dict(kernel=name.replace("fwd", "fwd+bwd") + " (torch SDPA)", shape=f"{H}x{S}x{S}x{D}", ms=lib,
                             tflops=3.5 * fl / lib / 1e9, frac_of_peak=3.5 * fl / lib / 1e9 / peaks["bf16_tflops"],
                             lib_ms=lib, lib_tflops=3.5 * fl / lib / 1e9, vs_lib=1.0, lib_name="itself"))
        except Exception as e:  # the library may not capture or may not take this head size
            print(f"torch SDPA row skipped: {type(e).__name__}: {e}")

    attention_row("attention fwd causal gptj", 2048, 16, 256)
    attention_row("attention fwd causal gptj tp4", 2048, 4, 256)

    def mem_row(name, fn, nbytes):
        if not want(name):
            return
        ms = time_ms(fn, iters=args.iters)
        rows.append(dict(kernel=name, ms=ms, gbs=nbytes / ms / 1e6, frac_of_peak=nbytes / ms / 1e6 / peaks["hbm_gbs"]))

    x = torch.randn(2048, 16384, device="cuda", dtype=bf)
    g = torch.randn_like(x)
    mem_row("gelu fwd 2048x16384", lambda: nat.gelu_cuda(x), 2 * x.numel() * 2)
    mem_row("gelu bwd 2048x16384", lambda: nat.gelu_grad_cuda(x, g), 3 * x.numel() * 2)
    h = torch.randn(8192, 4096, device="cuda", dtype=bf)
    w = torch.randn(4096, device="cuda", dtype=bf)
    b = torch.randn(4096, device="cuda", dtype=bf)
    gh = torch.randn_like(h)
    y, mean, rstd = nat.layer_norm_cuda(h, w, b, 1e-5)
    mem_row("layer_norm fwd 8192x4096", lambda: nat.layer_norm_cuda(h, w, b, 1e-5), 2 * h.numel() * 2)
    mem_row("layer_norm bwd 8192x4096", lambda: nat.layer_norm_grad_cuda(h, w, mean, rstd, gh), 3 * h.numel() * 2)
    n = 1 << 27
    pw = torch.randn(n, device="cuda", dtype=bf)
    pg = torch.randn(n, device="cuda")
    pm, pv, pmaster = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), pw.float()
    step = torch.zeros((), device="cuda")
    mem_row("adam 128M params (bf16 w, fp32 g/m/v/master)",
            lambda: nat.adam_cuda(pw, pg, pm, pv, step, pmaster, has_step=True, has_master=True, bias_correction=True,
                                  lr=1e-4, beta1=0.9, beta2=0.95, epsilon=1e-5, weight_decay=0.01, grad_scale=1.0,
                                  _tensor_scalars=()), n * (2 + 4 + 4 * 2 + 4 * 2 + 4 * 2 + 2))
    sc = torch.randn(16 * 2048, 2048, device="cuda", dtype=bf)
    lse = torch.empty(16 * 2048, device="cuda")
    mem_row("attn softmax fwd 16x2048x2048",
            lambda: nat._check(nat._sm_fwd(sc.data_ptr(), lse.data_ptr(), 16 * 2048, 2048, 2048, 0.0625, 1, 2,
                                           nat._stream()), "sm"), 2 * sc.numel() * 2)
    lg = torch.randn(2048, 50400, device="cuda", dtype=bf)
    lab = torch.randint(0, 50400, (2048,), device="cuda", dtype=torch.int32)
    one = torch.ones((), device="cuda")
    mem_row("cross-entropy fwd+bwd 2048x50400", lambda: nat.ce_with_grad_cuda(lg, lab, one, None, "mean"),
            2 * lg.numel() * 2)
    # ---- token-by-token decoding kernels (batch 16; GPT-J-6B shape at TP1 and at TP8) ----------------------------------
    from popxl_addons_b200.layers.linear_gq import interleave_scale_zero
    from popxl_addons_b200.models.generator import quantize_rows

    def small_row(name, fn, nbytes):
        """Kernels of a few microseconds: timed as replayed graph launches (device time only)."""
        if not want(name):
            return
        ms = graph_time_ms(fn)
        rows.append(dict(kernel=name + " [graph replay]", ms=ms, gbs=nbytes / ms / 1e6,
                         frac_of_peak=nbytes / ms / 1e6 / peaks["hbm_gbs"]))

    def gq_row(name, N, K, act_from=None):
        if not want(name):
            return
        # several weight sets used round-robin so that consecutive replayed launches do not find their weights in L2
        sets = []
        for _ in range(max(1, min(8, int(300e6 // (N * K // 2))))):
            wq = torch.randn(N, K, device="cuda") * 0.02
            packed, scale, zero = quantize_rows(wq, 64)
            sets.append((packed.view(torch.uint16), interleave_scale_zero(scale.half(), zero.half())))
        xin = torch.randn(16, K, device="cuda", dtype=bf)
        nbytes = N * K // 2 + sets[0][1].numel() * 2 + xin.numel() * 2 + 16 * N * 2
        for ctas in (None, 148, 74):
            state = {"i": 0}

            def fn():
                pk, sz = sets[state["i"] % len(sets)]
                state["i"] += 1
                return nat.gq_gemm_small_m(xin, pk, sz, None, None, act_from_col=act_from, ctas=ctas)

            small_row(f"{name} ctas={ctas or 'default'}", fn, nbytes)

    gq_row("gq gemm M=16 [qkv|fc_in] tp1 28672x4096", 28672, 4096, 12288)
    gq_row("gq gemm M=16 [out|fc_out] tp1 4096x20480", 4096, 20480)
    gq_row("gq gemm M=16 [qkv|fc_in] tp8 3584x4096", 3584, 4096, 1536)
    gq_row("gq gemm M=16 [out|fc_out] tp8 4096x2560", 4096, 2560)
    for heads, tag in ((16, "tp1"), (2, "tp8")):
        name = f"attn decode B=16 H={heads} D=256 len=576 {tag}"
        if want(name):
            qkv = torch.randn(16, 3 * heads * 256, device="cuda", dtype=bf)
            kc = torch.randn(16, heads, 640, 256, device="cuda", dtype=bf)
            vc = torch.randn_like(kc)
            pos = torch.tensor(575, dtype=torch.int32, device="cuda")
            small_row(name, lambda: nat.attention_decode_packed_cuda(qkv, kc, vc, pos, heads, 256, 0.0625),
                      2 * 16 * heads * 576 * 256 * 2)
    if want("add_layer_norm 16x4096"):
        xr = torch.randn(16, 4096, device="cuda", dtype=bf)
        dl = torch.randn_like(xr)
        small_row("add_layer_norm 16x4096",
                  lambda: nat.add_layer_norm_cuda(xr, dl, w, b, has_delta=True, has_bias=False, eps=1e-5), 4 * xr.numel() * 2)
    nat.check_gemm_errors()
    print(f"peaks ({src}): hbm {peaks['hbm_gbs']} GB/s, bf16 {peaks['bf16_tflops']} TFLOP/s")
    for r in rows:
        if "tflops" in r:
            print(f"{r['kernel']:38s} {r['shape']:>22s} {r['ms']:8.3f} ms {r['tflops']:8.1f} TF "
                  f"({r['frac_of_peak']*100:5.1f}% of {src}) | {r.get('lib_name', 'cuBLAS')} {r['lib_ms']:8.3f} ms "
                  f"{r['lib_tflops']:8.1f} TF | speed against it {r['vs_lib']:.2f}x")
        else:
            print(f"{r['kernel']:62s} {r['ms']:8.3f} ms {r['gbs']:8.1f} GB/s ({r['frac_of_peak']*100:5.1f}% of {src})")
    if args.out:
        json.dump(rows, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
