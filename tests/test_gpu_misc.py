"""The smaller CUDA ops (FP8 casts and GEMM, FP8 scale search, dense x CSR, embedding gather / scatter, row statistics of
the sharded LayerNorm and cross-entropy) against the fp32 PyTorch reference of the same op."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from popxl_addons_b200.ops import native

    return native


def _ref(name):
    from popxl_addons_b200.xl.opdef import OPS
    import popxl_addons_b200.xl.ops  # noqa: F401

    return OPS[name].impl


@pytest.mark.parametrize("fmt", ["float8_143", "float8_152"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_pow2scale_casts(nat, fmt, dtype):
    from popxl_addons_b200 import xl

    torch.manual_seed(0)
    x = (torch.randn(1000, 33, device="cuda") * 3).to(dtype)
    dt = getattr(xl, fmt)
    for ls in (torch.tensor(3, dtype=torch.int32, device="cuda"), torch.tensor(-2.0, device="cuda")):
        y = nat.pow2scale_cast_to_fp8_cuda(x, ls, dt)
        want = _ref("pow2scale_cast_to_fp8")(x, ls, dt)
        assert y is not NotImplemented and y.dtype == want.dtype
        torch.testing.assert_close(y.float(), want.float(), rtol=0, atol=0)
        back = nat.pow2scale_cast_from_fp8_cuda(y, -ls, xl.float16 if dtype != torch.float32 else xl.float32)
        want_back = _ref("pow2scale_cast_from_fp8")(want, -ls, xl.float16 if dtype != torch.float32 else xl.float32)
        torch.testing.assert_close(back.float(), want_back.float(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 384), (2048, 1024, 4096)])
@pytest.mark.parametrize("fa,fb", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
def test_fp8_gemm(nat, M, N, K, fa, fb):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda").to(fa)
    b_t = torch.randn(N, K, device="cuda").to(fb)
    ls = torch.tensor(-3, dtype=torch.int32, device="cuda")
    y = nat.gemm_fp8(a, b_t, out_dtype=torch.float32, log2_scale=ls)
    assert y is not NotImplemented
    want = (a.float() @ b_t.float().t()) * 0.125
    torch.testing.assert_close(y, want, rtol=1e-3, atol=1e-2 * np.sqrt(K / 128))
    nat.check_gemm_errors()
    # through the op: (K, N) right operand as LinearFP8 holds it
    from popxl_addons_b200 import xl

    y2 = nat.matmul_pow2scaled_cuda(a, b_t.t().contiguous(), ls, xl.bfloat16)
    torch.testing.assert_close(y2.float(), want, rtol=2e-2, atol=2e-2 * np.sqrt(K / 128) * 4)


@pytest.mark.parametrize("fmt", ["float8_143", "float8_152"])
def test_fp8_mse_scale_matches_the_host_algorithm(nat, fmt):
    from popxl_addons_b200.ops.fp8_mse_scale import fp8_mse_scale_reference

    torch.manual_seed(2)
    for scale, dtype, mant in ((1.0, torch.float32, 23), (300.0, torch.float16, 10), (1e-3, torch.bfloat16, 7)):
        x = (torch.randn(100_000, device="cuda") * scale).to(dtype)
        for _ in range(2):  # the scratch histogram must come back zeroed
            got = nat.fp8_mse_scale_cuda(x, fmt, mant)
            want = fp8_mse_scale_reference(x.cpu(), fmt, mant)
            assert int(got) == int(want)


def test_dense_csr_matmul(nat):
    from scipy.sparse import random as sprandom

    rs = np.random.RandomState(0)
    K, N, M = 96, 200, 37
    sp = sprandom(K, N, density=0.1, format="csr", random_state=rs, dtype=np.float32)
    x = torch.randn(2, M, K, device="cuda")
    args = [torch.tensor(sp.indptr.astype(np.int32), device="cuda"), torch.tensor(sp.indices.astype(np.int32), device="cuda"),
            torch.tensor(sp.data.astype(np.float32), device="cuda")]
    y = nat.dense_csr_matmul_cuda(x, *args, K, N)
    want = x.cpu().numpy() @ sp.toarray()
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_rows_and_gradient(nat, dtype):
    torch.manual_seed(3)
    table = torch.randn(300, 128, device="cuda").to(dtype)
    idx = torch.randint(-20, 330, (4, 50), device="cuda", dtype=torch.int32)
    out = nat.gather_cuda(table, idx, 0, True)
    want = _ref("gather")(table, idx, 0, True)
    torch.testing.assert_close(out, want)
    g = torch.randn(4, 50, 128, device="cuda").to(dtype)
    dw = nat.gather_grad_cuda(g, idx, 0, True, (300, 128))
    want_dw = _ref("gather_grad")(g, idx, 0, True, (300, 128))
    torch.testing.assert_close(dw.float(), want_dw.float(), rtol=2e-2, atol=2e-2)


def test_row_statistics_kernels(nat):
    torch.manual_seed(4)
    x = torch.randn(64, 1000, device="cuda").bfloat16()
    stats = nat.row_sum_sumsq(x)
    torch.testing.assert_close(stats[0], x.float().sum(-1), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(stats[1], (x.float() ** 2).sum(-1), rtol=1e-3, atol=1e-2)
    w, b = torch.randn(1000, device="cuda").bfloat16(), torch.randn(1000, device="cuda").bfloat16()
    y, mean, rstd = nat.ln_apply_stats(x, stats, w, b, 1000, 1e-5)
    want = torch.nn.functional.layer_norm(x.float(), (1000,), w.float(), b.float(), 1e-5)
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=3e-2)
    # vocabulary-sharded cross-entropy kernels on two uneven "shards" of one device
    labels = torch.randint(0, 1000, (64,), device="cuda", dtype=torch.int32)
    shards, offs = [x[:, :600].contiguous(), x[:, 600:].contiguous()], [0, 600]
    stats = torch.stack([nat.ce_shard_stats(sh, labels, off) for sh, off in zip(shards, offs)])
    torch.testing.assert_close(stats[0, 0], shards[0].float().amax(-1))
    g = nat.ce_shard_combine(stats)
    torch.testing.assert_close(g[0], x.float().amax(-1))
    torch.testing.assert_close(g[1], torch.exp(x.float() - g[0][:, None]).sum(-1), rtol=1e-4, atol=1e-4)
    want_loss = torch.nn.functional.cross_entropy(x.float(), labels.long(), reduction="none")
    scale = torch.full((64,), 0.5, device="cuda")
    xf = x.float().requires_grad_(True)
    (torch.nn.functional.cross_entropy(xf, labels.long(), reduction="none") * 0.5).sum().backward()
    for sh, off in zip(shards, offs):
        dx, loss = nat.ce_shard_grad_loss(sh, g[0], g[1], g[2], labels, off, scale)
        torch.testing.assert_close(loss, want_loss, rtol=1e-3, atol=1e-3)
        torch.testing.assert_close(dx.float(), xf.grad[:, off:off + sh.shape[1]], rtol=2e-2, atol=2e-3)
        nls, loss16 = nat.ce_shard_nls(sh, g[0], g[1], g[2])
        want_nls = -torch.log_softmax(x.float(), -1)[:, off:off + sh.shape[1]]
        torch.testing.assert_close(nls.float(), want_nls, rtol=2e-2, atol=5e-2)
        back = nat.ce_nls_grad(nls, labels, off, scale.to(nls.dtype))
        torch.testing.assert_close(back.float(), xf.grad[:, off:off + sh.shape[1]], rtol=5e-2, atol=5e-3)


@pytest.mark.parametrize("shape,axes,dtype", [((2048, 4096), [0], torch.bfloat16), ((300, 1024), [0], torch.float32),
                                              ((2, 128, 264), [0, 1], torch.float16), ((2048, 16384), [0], torch.bfloat16)])
def test_column_sums(nat, shape, axes, dtype):
    """`sum` over the leading axes (bias gradients) against an fp32 sum of the same values; two launches give the
    same bits (fixed order of additions)."""
    torch.manual_seed(3)
    a = torch.randn(*shape, device="cuda").to(dtype)
    before = nat.LAUNCHES["by_kernel"].get("col_sum", 0)
    got = nat.sum_cuda(a, axes, False)
    assert got is not NotImplemented and nat.LAUNCHES["by_kernel"].get("col_sum", 0) == before + 1
    want = a.float().sum(dim=axes)
    rows = a.numel() // want.numel()
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype] * (rows ** 0.5)
    torch.testing.assert_close(got.float(), want, rtol=1e-2 if dtype != torch.float32 else 1e-5, atol=tol)
    assert torch.equal(got, nat.sum_cuda(a, axes, False))
    assert nat.sum_cuda(a, [len(shape) - 1], False) is NotImplemented  # trailing axes stay on the library path
