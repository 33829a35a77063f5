"""Every CUDA kernel against the plain-PyTorch fp32 reference of the same op (the op's own reference implementation,
evaluated in fp32 on the same inputs)."""
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from popxl_addons_b200.ops import native

    return native


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-4, atol=1e-5)


def _ref(name):
    from popxl_addons_b200.xl.opdef import OPS
    import popxl_addons_b200.xl.ops  # noqa: F401

    return OPS[name].impl


DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("approx", ["none", "tanh"])
def test_gelu(nat, dtype, approx):
    torch.manual_seed(0)
    x = torch.randn(1000, 517, device="cuda", dtype=dtype)
    g = torch.randn_like(x)
    y = nat.gelu_cuda(x, approximate=approx)
    dx = nat.gelu_grad_cuda(x, g, approximate=approx)
    torch.testing.assert_close(y.float(), _ref("gelu")(x.float(), approx), **_tol(dtype))
    torch.testing.assert_close(dx.float(), _ref("gelu_grad")(x.float(), g.float(), approx), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_silu(nat, dtype):
    torch.manual_seed(1)
    a = torch.randn(64, 1024, device="cuda", dtype=dtype)
    b = torch.randn_like(a)
    g = torch.randn_like(a)
    torch.testing.assert_close(nat.swiglu_cuda(a, b).float(), _ref("swiglu")(a.float(), b.float()), **_tol(dtype))
    da, db = nat.swiglu_grad_cuda(a, b, g)
    ra, rb = _ref("swiglu_grad")(a.float(), b.float(), g.float())
    torch.testing.assert_close(da.float(), ra, **_tol(dtype))
    torch.testing.assert_close(db.float(), rb, **_tol(dtype))
    torch.testing.assert_close(nat.swish_cuda(a).float(), _ref("swish")(a.float()), **_tol(dtype))
    torch.testing.assert_close(nat.swish_grad_cuda(a, g).float(), _ref("swish_grad")(a.float(), g.float()), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,cols", [(300, 768), (300, 4096), (40, 4096), (2051, 2048)])
def test_layer_norm_fwd_bwd(nat, dtype, rows, cols):
    """Forward and backward against the fp32 reference: rows shorter and longer than one register tiling, fewer rows
    than CTAs, a row count that is no multiple of the grid."""
    torch.manual_seed(2)
    x = torch.randn(rows, cols, device="cuda", dtype=dtype) * 2 + 0.5
    w = torch.randn(cols, device="cuda", dtype=dtype)
    b = torch.randn(cols, device="cuda", dtype=dtype)
    g = torch.randn_like(x)
    y, mean, rstd = nat.layer_norm_cuda(x, w, b, 1e-5)
    ry, rmean, rrstd = _ref("layer_norm")(x.float(), w.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), ry, **_tol(dtype))
    torch.testing.assert_close(mean, rmean, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(rstd, rrstd, rtol=1e-4, atol=1e-4)
    dx, dw, db = nat.layer_norm_grad_cuda(x, w, mean, rstd, g)
    rdx, rdw, rdb = _ref("layer_norm_grad")(x.float(), w.float(), rmean, rrstd, g.float())
    torch.testing.assert_close(dx.float(), rdx, **_tol(dtype))
    big = dict(rtol=3e-2, atol=0.3 * max(1.0, (rows / 300) ** 0.5)) if dtype != torch.float32 else dict(rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(dw.float(), rdw, **big)
    torch.testing.assert_close(db.float(), rdb, **big)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_fwd_bwd(nat, dtype):
    torch.manual_seed(3)
    x = torch.randn(257, 4096, device="cuda", dtype=dtype)
    w = torch.randn(4096, device="cuda", dtype=dtype)
    g = torch.randn_like(x)
    y, rstd = nat.rms_norm_cuda(x, w, 1e-5)
    ry, rr = _ref("rms_norm")(x.float(), w.float(), 1e-5)
    torch.testing.assert_close(y.float(), ry, **_tol(dtype))
    dx, dw = nat.rms_norm_grad_cuda(x, w, rstd, g)
    rdx, rdw = _ref("rms_norm_grad")(x.float(), w.float(), rr, g.float())
    torch.testing.assert_close(dx.float(), rdx, **_tol(dtype))
    big = dict(rtol=3e-2, atol=0.3) if dtype != torch.float32 else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(dw.float(), rdw, **big)


@pytest.mark.parametrize("wdtype,mdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                           (torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16)])
def test_adam_matches_torch_adamw(nat, wdtype, mdtype):
    torch.manual_seed(4)
    n = 100003
    w0 = torch.randn(n, device="cuda")
    master = w0.clone() if wdtype != torch.float32 else None
    w = w0.to(wdtype)
    m = torch.zeros(n, device="cuda", dtype=mdtype)
    v = torch.zeros(n, device="cuda")
    step = torch.zeros((), device="cuda")
    ref_w = w0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_w], lr=1e-2, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.1)
    for i in range(3):
        g = torch.randn(n, device="cuda")
        args = [w, g.to(wdtype) if i % 2 else g, m, v, step] + ([master] if master is not None else [])
        out = nat.adam_cuda(*args, has_step=True, has_master=master is not None, bias_correction=True, lr=1e-2,
                            beta1=0.9, beta2=0.95, epsilon=1e-6, weight_decay=0.1, grad_scale=1.0, _tensor_scalars=())
        assert out is w
        ref_w.grad = (g.to(wdtype).float() if i % 2 else g)
        opt.step()
    assert float(step) == 3.0
    got = master if master is not None else w
    tol = dict(rtol=1e-4, atol=1e-5) if mdtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(got.float(), ref_w.detach(), **tol)


def test_sgd_and_accumulate_mean_and_sumsq(nat):
    torch.manual_seed(5)
    n = 4099
    w = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    buf = torch.zeros(n, device="cuda")
    ref = _ref("sgd_fused_")(w.clone(), g, buf.clone(), has_momentum=True, lr=0.1, momentum=0.9, weight_decay=0.01,
                             grad_scale=0.5, _tensor_scalars=())
    nat.sgd_cuda(w, g, buf, has_momentum=True, lr=0.1, momentum=0.9, weight_decay=0.01, grad_scale=0.5,
                 _tensor_scalars=())
    torch.testing.assert_close(w, ref, rtol=1e-5, atol=1e-6)
    acc = torch.zeros(n, device="cuda")
    step = torch.zeros((), device="cuda")
    xs = [torch.randn(n, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    for x in xs:
        nat.accumulate_mean_cuda(acc, x, step, step=None, _tensor_scalars=("step",))
        step += 1
    torch.testing.assert_close(acc, torch.stack([x.float() for x in xs]).mean(0), rtol=1e-5, atol=1e-6)
    t = torch.randn(1 << 20, device="cuda", dtype=torch.bfloat16)
    s = nat.grad_sumsq_cuda(t, torch.tensor(0.25, device="cuda"))
    torch.testing.assert_close(s, (t.float() ** 2).sum() * 0.25, rtol=1e-4, atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotary(nat, dtype):
    from popxl_addons_b200.ops.rotary_pos_embed import trig_tables

    torch.manual_seed(6)
    x = torch.randn(2, 4, 128, 256, device="cuda", dtype=dtype)
    sin, cos = trig_tables(128, 64)
    sin = torch.tensor(sin[None], device="cuda", dtype=dtype)
    cos = torch.tensor(cos[None], device="cuda", dtype=dtype)
    for inverse in (False, True):
        y = nat.rotary_cuda(x, sin, cos, 64, inverse)
        ref = _ref("rotary_pos_embed")(x.float(), sin.float(), cos.float(), 64, inverse)
        torch.testing.assert_close(y.float(), ref, **_tol(dtype))


def test_group_quantize_decompress(nat):
    from popxl_addons_b200.ops.group_quantize_decompress import (group_quantize_compress_numpy,
                                                                group_quantize_decompress_numpy)

    rng = np.random.RandomState(7)
    w = rng.randn(512, 1024).astype(np.float16)
    packed, scale, bias = group_quantize_compress_numpy(w, 64, -1)
    ref = group_quantize_decompress_numpy(packed, scale, bias)
    from popxl_addons_b200.xl.dtypes import to_torch

    out = nat.gq_decompress_cuda(to_torch(packed).cuda(), torch.tensor(scale).cuda(), torch.tensor(bias).cuda())
    np.testing.assert_allclose(out.float().cpu().numpy(), ref.astype(np.float32), atol=1e-2)
    assert np.abs(ref.astype(np.float32) - w.astype(np.float32)).max() < 0.5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_fused(nat, dtype):
    torch.manual_seed(8)
    logits = torch.randn(64, 50400, device="cuda", dtype=dtype) * 3
    labels = torch.randint(0, 50400, (64,), device="cuda", dtype=torch.int32)
    labels[5] = -100
    loss, dl = nat.ce_with_grad_cuda(logits, labels, torch.tensor(2.0, device="cuda"), -100, "mean")
    ref_logits = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_logits, labels.long(), ignore_index=-100)
    (ref * 2.0).backward()
    torch.testing.assert_close(loss.float(), ref.detach(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dl.float(), ref_logits.grad, rtol=2e-2, atol=1e-4)


# ---- tcgen05 GEMM -------------------------------------------------------------------------------------------------------


def _gemm_check(nat, a, b, **kw):
    out = nat.gemm(a, b, **kw)
    assert out is not NotImplemented
    torch.cuda.synchronize()
    nat.check_gemm_errors()
    return out


def _gemm_tol(K, dtype=torch.bfloat16, sigma_a=1.0, sigma_b=1.0):
    """Bound for a 16-bit result of an fp32-accumulated product of N(0, sigma) operands: the entries have standard
    deviation sqrt(K) sigma_a sigma_b, rounding them to the output type costs half a unit in the last place (2^-9 for
    bf16, 2^-12 for fp16) of their magnitude, and the fp32 accumulation order adds far less. Two bits of slack."""
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    return dict(rtol=ulp, atol=ulp * math.sqrt(K) * sigma_a * sigma_b)


@pytest.fixture(params=["cta_pairs", "single_cta"])
def gemm_kernel(request, nat):
    """Runs a GEMM test on both tcgen05 kernels: CTA pairs (default for plain products) and the single-CTA kernel."""
    old = nat._GEMM_CTA_PAIRS
    nat._GEMM_CTA_PAIRS = request.param == "cta_pairs"
    yield request.param
    nat._GEMM_CTA_PAIRS = old


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 128), (2048, 4096, 1024), (200, 328, 136),
                                   (16, 4096, 4096), (1000, 50400, 512)])
def test_gemm_k_major_a_mn_major_b(nat, gemm_kernel, dtype, M, N, K):
    """Forward layout: x (M,K) row-major @ w (K,N) row-major."""
    torch.manual_seed(10)
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(K, N, device="cuda", dtype=dtype)
    out = _gemm_check(nat, a, b)
    ref = a.float() @ b.float()
    torch.testing.assert_close(out.float(), ref, **_gemm_tol(K, dtype))


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (2048, 1024, 4096), (136, 200, 328)])
def test_gemm_all_operand_layouts(nat, gemm_kernel, M, N, K):
    torch.manual_seed(11)
    dtype = torch.bfloat16
    a_km = torch.randn(M, K, device="cuda", dtype=dtype)          # K-major A
    a_mn = torch.randn(K, M, device="cuda", dtype=dtype).t()       # MN-major A (view)
    b_mn = torch.randn(K, N, device="cuda", dtype=dtype)          # MN-major B
    b_km = torch.randn(N, K, device="cuda", dtype=dtype).t()       # K-major B (view)
    for a in (a_km, a_mn):
        for b in (b_mn, b_km):
            out = _gemm_check(nat, a, b)
            ref = a.float() @ b.float()
            torch.testing.assert_close(out.float(), ref, **_gemm_tol(K))


def test_gemm_batched_and_epilogues(nat, gemm_kernel):
    torch.manual_seed(12)
    dtype = torch.bfloat16
    q = torch.randn(6, 256, 128, device="cuda", dtype=dtype)
    k = torch.randn(6, 384, 128, device="cuda", dtype=dtype)
    s = _gemm_check(nat, q, k.transpose(-1, -2))
    torch.testing.assert_close(s.float(), q.float() @ k.float().transpose(-1, -2), rtol=2e-2, atol=0.3)
    a = torch.randn(512, 256, device="cuda", dtype=dtype)
    b = torch.randn(256, 384, device="cuda", dtype=dtype)
    bias = torch.randn(384, device="cuda", dtype=dtype)
    out = _gemm_check(nat, a, b, bias=bias, act=1)
    ref = torch.nn.functional.gelu(a.float() @ b.float() + bias.float())
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=0.3)
    # fp32 output, accumulate and running mean
    acc = torch.ones(512, 384, device="cuda")
    _gemm_check(nat, a, b, out=acc, accumulate=1)
    torch.testing.assert_close(acc, 1.0 + a.float() @ b.float(), rtol=1e-3, atol=1e-2)
    mean = torch.zeros(512, 384, device="cuda")
    step = torch.zeros((), device="cuda")
    parts = []
    for i in range(3):
        ai = torch.randn(512, 256, device="cuda", dtype=dtype)
        parts.append(ai.float() @ b.float())
        _gemm_check(nat, ai, b, out=mean, accumulate=2, step=step)
        step += 1
    torch.testing.assert_close(mean, torch.stack(parts).mean(0), rtol=1e-3, atol=1e-2)


def test_attention_forward_backward(nat):
    torch.manual_seed(13)
    B, H, S, D = 2, 4, 512, 128
    q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16) * 0.5 for _ in range(3))
    do = torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    o, lse = nat.attention_cuda(q, k, v, True, scale)
    ro, rlse = _ref("attention")(q.float(), k.float(), v.float(), True, scale)
    torch.testing.assert_close(o.float(), ro, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(lse, rlse, rtol=1e-2, atol=2e-2)
    dq, dk, dv = nat.attention_grad_cuda(q, k, v, o, lse, do, True, scale)
    rdq, rdk, rdv = _ref("attention_grad")(q.float(), k.float(), v.float(), ro, rlse, do.float(), True, scale)
    for got, ref in ((dq, rdq), (dk, rdk), (dv, rdv)):
        torch.testing.assert_close(got.float(), ref, rtol=5e-2, atol=5e-2)
    nat.check_gemm_errors()


@pytest.mark.parametrize("B,S,H,D,causal,dtype", [(2, 256, 2, 64, True, torch.bfloat16), (1, 384, 2, 128, True, torch.float16),
                                                  (1, 512, 1, 256, True, torch.bfloat16), (1, 300, 2, 64, False, torch.bfloat16),
                                                  (2, 200, 1, 256, True, torch.bfloat16)])
def test_single_kernel_attention_forward(nat, B, S, H, D, causal, dtype):
    """Heads as column windows of a packed (tokens, 3*H*D) matrix; output and log-sum-exp against fp32 PyTorch."""
    torch.manual_seed(21)
    hd = H * D
    qkv = (torch.randn(B * S, 3 * hd, device="cuda") * 0.7).to(dtype)
    scale = 1.0 / math.sqrt(D)
    res = nat.flash_attention_fwd(qkv, 0, hd, 2 * hd, B, S, H, D, scale, causal)
    assert res is not NotImplemented
    out, lse = res
    nat.check_gemm_errors()
    q, k, v = (qkv[:, i * hd:(i + 1) * hd].float().reshape(B, S, H, D).transpose(1, 2) for i in range(3))
    s = q @ k.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    want = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B * S, hd)
    torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(lse, torch.logsumexp(s, -1), rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("B,S,H,D,rot,dtype", [(1, 256, 2, 64, 32, torch.bfloat16), (2, 384, 2, 128, 0, torch.float16),
                                                (1, 512, 2, 256, 64, torch.bfloat16), (1, 2048, 1, 256, 64, torch.bfloat16),
                                                (2, 200, 1, 256, 0, torch.bfloat16)])
def test_attention_on_packed_qkv_forward_and_fused_backward(nat, B, S, H, D, rot, dtype):
    """`attention_qkv` and its gradient as the training step runs them (rotary in place, single-kernel forward, backward
    with scores, dP and the dQ accumulator on chip + two causal GEMMs) against the fp32 reference of the same ops."""
    from popxl_addons_b200.ops.rotary_pos_embed import trig_tables

    torch.manual_seed(31)
    hd = H * D
    qkv = (torch.randn(B * S, 3 * hd, device="cuda") * 0.6).to(dtype)
    dout = (torch.randn(B * S, hd, device="cuda") * 0.5).to(dtype)
    sin_np, cos_np = trig_tables(S, rot if rot else 2)
    sin, cos = (torch.tensor(t[None]).to(dtype).cuda() for t in (sin_np, cos_np))
    scale = 1.0 / math.sqrt(D)
    kw = dict(seq_len=S, n_heads=H, head_dim=D, rotary_dim=rot, causal=True, scale=scale)
    saved = nat._FLASH_ATTENTION
    nat._FLASH_ATTENTION = "1"
    try:
        out, qkv_rot, lse = nat.attention_qkv_cuda(qkv, sin, cos, inplace=False, **kw)
    finally:
        nat._FLASH_ATTENTION = saved
    r_out, r_rot, r_lse = _ref("attention_qkv")(qkv.float(), sin.float(), cos.float(), inplace=False, **kw)
    torch.testing.assert_close(out.float(), r_out, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(lse, r_lse, rtol=1e-3, atol=1e-2)
    before = nat.LAUNCHES["by_kernel"].get("attn_bwd_dq_tcgen05", 0)
    dqkv = nat.attention_qkv_grad_cuda(qkv_rot, lse, dout, sin, cos, out, **kw)
    assert dqkv is not NotImplemented
    nat.check_gemm_errors()
    assert nat.LAUNCHES["by_kernel"].get("attn_bwd_dq_tcgen05", 0) == before + 1, "the fused backward kernel did not run"
    r_dqkv = _ref("attention_qkv_grad")(r_rot, r_lse, dout.float(), sin.float(), cos.float(), **kw)
    # gradients are sums over up to S keys of 16-bit products: compare relative to the largest entry of each third
    for i, name in enumerate(("dq", "dk", "dv")):
        got, want = dqkv[:, i * hd:(i + 1) * hd].float(), r_dqkv[:, i * hd:(i + 1) * hd]
        err = (got - want).abs().max() / want.abs().max()
        assert err < 3e-2, f"{name}: relative error {float(err):.4f}"
    # the GEMM-based backward (scores recomputed, two softmax kernels) must agree as well
    saved_bwd, nat._FLASH_ATTENTION_BWD = nat._FLASH_ATTENTION_BWD, False
    try:
        dqkv2 = nat.attention_qkv_grad_cuda(qkv_rot, lse, dout, sin, cos, out, **kw)
    finally:
        nat._FLASH_ATTENTION_BWD = saved_bwd
    err = (dqkv2.float() - r_dqkv).abs().max() / r_dqkv.abs().max()
    assert err < 3e-2, f"GEMM-based backward: relative error {float(err):.4f}"
    # few heads: the keys of a query block were divided over several CTAs (partial results merged by the last to finish);
    # the same kernels with every query block in one CTA must give the same values up to the rounding of the partials
    split = [nat._attention_split(kind, fn, B, S, H, D, True, qkv.device)[0]
             for kind, fn in (("fwd", nat._attn_plan), ("bwd", nat._attn_bwd_plan))]
    if S >= 512:
        assert all(c > 0 for c in split), split
    saved_split, saved_plans = nat._ATTN_SPLIT, dict(nat._ATTN_PLANS)
    nat._ATTN_SPLIT, nat._FLASH_ATTENTION = False, "1"
    nat._ATTN_PLANS.clear()
    try:
        out1, _, lse1 = nat.attention_qkv_cuda(qkv, sin, cos, inplace=False, **kw)
        dqkv1 = nat.attention_qkv_grad_cuda(qkv_rot, lse, dout, sin, cos, out, **kw)
    finally:
        nat._ATTN_SPLIT, nat._FLASH_ATTENTION = saved_split, saved
        nat._ATTN_PLANS.clear()
        nat._ATTN_PLANS.update(saved_plans)
    nat.check_gemm_errors()
    torch.testing.assert_close(out.float(), out1.float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(lse, lse1, rtol=1e-4, atol=1e-3)
    err = (dqkv.float() - dqkv1.float()).abs().max() / dqkv1.float().abs().max()
    assert err < 1e-2, f"split against whole: relative error {float(err):.4f}"


@pytest.mark.parametrize("M,N,K,batch,ta,tb,dtype", [
    (256, 256, 64, 1, False, False, torch.bfloat16),      # one tile, one k-block
    (512, 512, 512, 1, False, False, torch.bfloat16),     # the ring wraps (8 k-blocks over 6 stages)
    (384, 640, 200, 1, False, False, torch.float16),      # ragged M (peer half empty), N and K
    (512, 768, 256, 1, True, False, torch.bfloat16),      # A stored (K, M)
    (512, 768, 256, 1, False, True, torch.bfloat16),      # B stored (N, K)
    (512, 768, 256, 1, True, True, torch.bfloat16),
    (300, 264, 128, 3, False, False, torch.bfloat16),     # batched
    (4096, 4096, 1024, 1, False, True, torch.bfloat16),   # more tiles than CTA pairs: both accumulator buffers cycle
])
@pytest.mark.parametrize("tile_n", [256, 128])
def test_cta_pair_gemm(nat, M, N, K, batch, ta, tb, dtype, tile_n, monkeypatch):
    """256 x 256 and 256 x 128 tiles on CTA pairs against an fp32 product; every epilogue form on one shape."""
    monkeypatch.setattr(nat, "_GEMM_PAIR_TILE_N", [tile_n])
    torch.manual_seed(5)
    lead = (batch,) if batch > 1 else ()
    a = torch.randn(*lead, K, M, device="cuda").to(dtype).transpose(-1, -2) if ta else torch.randn(*lead, M, K, device="cuda").to(dtype)
    b = torch.randn(*lead, N, K, device="cuda").to(dtype).transpose(-1, -2) if tb else torch.randn(*lead, K, N, device="cuda").to(dtype)
    want = a.float() @ b.float()
    before = nat.LAUNCHES["by_kernel"].get("gemm2cta_tcgen05", 0)
    out = nat.gemm(a, b)
    assert out is not NotImplemented
    nat.check_gemm_errors()
    assert nat.LAUNCHES["by_kernel"].get("gemm2cta_tcgen05", 0) == before + 1, "the CTA-pair kernel did not run"
    torch.testing.assert_close(out.float(), want, **_gemm_tol(K, dtype))
    if (M, N, K) == (512, 512, 512):
        bias = torch.randn(N, device="cuda").to(dtype)
        got = nat.gemm(a, b, bias=bias, act=3, alpha=0.5, out_dtype=torch.float32)
        torch.testing.assert_close(got, torch.relu(0.5 * want + bias.float()), rtol=2e-2, atol=0.5)
        acc = torch.ones(M, N, device="cuda")
        nat.gemm(a, b, out=acc, accumulate=1)
        torch.testing.assert_close(acc, want + 1.0, rtol=2e-2, atol=0.5)
        step = torch.full((1,), 3.0, device="cuda")
        mean = torch.full((M, N), 4.0, device="cuda")
        nat.gemm(a, b, out=mean, accumulate=2, step=step)
        torch.testing.assert_close(mean, 4.0 * 0.75 + want * 0.25, rtol=2e-2, atol=0.5)
        nat.check_gemm_errors()


def test_bounded_wait_on_a_peer_gives_up_and_reports(nat):
    """Failure detection on the device without a fault: a barrier whose peer never signals (a flag nothing sets) must
    run out of its poll budget, record the reason in the status word and return; the context stays usable."""
    pad_a = torch.zeros(256, dtype=torch.int32, device="cuda")  # this rank's signal pad
    pad_b = torch.zeros(256, dtype=torch.int32, device="cuda")  # stands for the silent peer's pad
    pads = torch.tensor([pad_a.data_ptr(), pad_b.data_ptr()], dtype=torch.int64, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    nat.set_comm_spin_limit(1 << 12)
    try:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        nat._check(nat._symm_barrier(pads.data_ptr(), 0, 2, 4, err.data_ptr(), nat._stream()), "symm_barrier")
        end.record()
        torch.cuda.synchronize()
    finally:
        nat.set_comm_spin_limit(0)
    assert int(err.item()) == 102  # "a peer's signal never arrived"
    assert start.elapsed_time(end) < 1000.0
    # the signal this rank sent did arrive at the (silent) peer's pad: slot (channel 4, sender 0)
    assert int(pad_b[4 * 2 + 0].item()) == 1
    # and the context is intact: ordinary work still runs
    x = torch.randn(1024, 512, device="cuda").bfloat16()
    torch.testing.assert_close(nat.gelu_cuda(x, approximate="none").float(), torch.nn.functional.gelu(x.float()),
                               rtol=2e-2, atol=2e-2)


def test_matmul_add_accumulates_in_the_epilogue(nat):
    from popxl_addons_b200.parallel.passes import _matmul_add_cuda

    torch.manual_seed(7)
    a1, w1 = (torch.randn(512, 384, device="cuda") * 0.1).bfloat16(), (torch.randn(384, 640, device="cuda") * 0.1).bfloat16()
    a2, w2 = (torch.randn(512, 256, device="cuda") * 0.1).bfloat16(), (torch.randn(256, 640, device="cuda") * 0.1).bfloat16()
    c = nat.gemm(a1, w1)
    want = c.float() + a2.float() @ w2.float()
    got = _matmul_add_cuda(c, a2, w2)
    assert got is not NotImplemented and got.data_ptr() == c.data_ptr()
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)
