"""The wider popxl op surface (pooling, resize, scatter, reductions, histogram, ...) against PyTorch, values and
gradients, on the CPU backend."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops


def _run(build, *arrays, grads=True):
    """Trace `build(*tensors) -> tensor`, run it, and (if `grads`) its autodiff graph with an all-ones seed."""
    ir = popxl.Ir()
    with ir.main_graph:
        ins = [popxl.variable(a, name=f"in{i}") for i, a in enumerate(arrays)]
        g = ir.create_graph(build, *ins)
        info = ops.call_with_info(g, *ins)
        y = info.outputs[0]
        streams = [addons.host_store(y)]
        if grads:
            diff = [t for t, a in zip(g.inputs, arrays) if a.dtype == np.float32]
            gi = popxl.transforms.autodiff(g, grads_required=diff)
            seed = popxl.constant(np.ones(y.shape, np.float32))
            outs = ops.call(gi.graph, seed, inputs_dict=gi.inputs_dict(info))
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
            streams += [addons.host_store(o) for o in outs]
    with popxl.Session(ir, "cpu") as s:
        res = s.run({})
    return [np.asarray(res[st]) for st in streams]


def _torch(fn, *arrays):
    ts = [torch.tensor(a, requires_grad=a.dtype == np.float32) for a in arrays]
    y = fn(*ts)
    gs = torch.autograd.grad(y.sum(), [t for t in ts if t.requires_grad], allow_unused=True)
    return [y.detach().numpy()] + [None if g is None else g.numpy() for g in gs]


def _check(got, want, tol=1e-5):
    assert len(got) == len(want)
    for a, b in zip(got, want):
        np.testing.assert_allclose(a, b, rtol=tol, atol=tol)


rs = np.random.RandomState(0)
IMG = rs.randn(2, 3, 8, 10).astype(np.float32)


def test_pooling_and_resize():
    _check(_run(lambda x: ops.average_pool(x, (2, 2), (2, 2)), IMG), _torch(lambda x: F.avg_pool2d(x, 2, 2), IMG))
    _check(_run(lambda x: ops.average_pool(x, (3, 3), (1, 1), (1, 1, 1, 1)), IMG),
           _torch(lambda x: F.avg_pool2d(x, 3, 1, 1, count_include_pad=False), IMG))
    _check(_run(lambda x: ops.max_pool(x, (3, 2), (2, 1), (1, 0, 1, 0)), IMG),
           _torch(lambda x: F.max_pool2d(x, (3, 2), (2, 1), (1, 0)), IMG))
    # uneven padding: one extra row at the bottom only
    _check(_run(lambda x: ops.max_pool(x, (2, 2), (2, 2), (0, 0, 2, 0)), IMG),
           _torch(lambda x: F.max_pool2d(F.pad(x, (0, 0, 0, 2), value=float("-inf")), 2, 2), IMG))
    _check(_run(lambda x: ops.interpolate(x, (1, 1, 2, 2)), IMG),
           _torch(lambda x: F.interpolate(x, scale_factor=2, mode="nearest"), IMG))
    _check(_run(lambda x: ops.interpolate(x, (1, 1, 2, 1.5), mode="linear"), IMG),
           _torch(lambda x: F.interpolate(x, size=(16, 15), mode="bilinear", align_corners=False), IMG))
    with pytest.raises(ValueError):
        _run(lambda x: ops.interpolate(x, (2, 1, 1, 1)), IMG)


def test_roi_align():
    from torchvision.ops import roi_align as tv

    rois = np.array([[0.5, 1.0, 6.0, 5.5], [2.0, 0.0, 9.0, 7.0], [1.0, 1.0, 4.0, 4.0]], np.float32)
    bidx = np.array([0, 1, 1], np.int32)
    got = _run(lambda x, r, b: ops.roi_align(x, r, b, (3, 2), 0.5, 2), IMG, rois, bidx)

    def want(x, r):
        boxes = torch.cat([torch.tensor(bidx).float()[:, None], r], 1)
        return tv(x, boxes, (3, 2), 0.5, 2, aligned=False)

    ref = _torch(want, IMG, rois)
    _check(got[:2], ref[:2], 1e-5)  # value and the gradient with respect to the feature map


def test_conv_transpose_and_batch_norm_inference():
    w = rs.randn(3, 4, 3, 3).astype(np.float32)
    _check(_run(lambda x, w: ops.conv_transpose(x, w, (2, 2), (1, 1, 1, 1), output_padding=(1, 1)), IMG, w),
           _torch(lambda x, w: F.conv_transpose2d(x, w, None, 2, 1, 1), IMG, w), 1e-4)
    sc, b, m = (rs.randn(3).astype(np.float32) for _ in range(3))
    v = rs.rand(3).astype(np.float32) + 0.5

    def want(x, sc, b):
        return F.batch_norm(x, torch.tensor(m), torch.tensor(v), sc, b, False, 0.0, 1e-5)

    got = _run(lambda x, sc, b: ops.batch_norm_inference(x, sc, b, popxl.constant(m), popxl.constant(v)), IMG, sc, b)
    _check(got, _torch(want, IMG, sc, b), 1e-4)


def test_scatter_tied_gather_subsample():
    t = rs.randn(6, 5).astype(np.float32)
    idx = np.stack([rs.permutation(6)[:3] for _ in range(5)], axis=1).astype(np.int32)
    val = rs.randn(3, 5).astype(np.float32)
    got = _run(lambda t, v, i: ops.scatter(t, 0, i, v), t, val, idx)
    want = _torch(lambda t, v: t.scatter(0, torch.tensor(idx).long(), v), t, val)
    _check(got, want)
    ids = np.array([0, 5, 2, 2], np.int32)
    _check(_run(lambda t, i: ops.tied_gather(t, i), t, ids), _torch(lambda t: t[torch.tensor(ids).long()], t))
    _check(_run(lambda t: ops.subsample(t, (2, 3)), t), _torch(lambda t: t[::2, ::3], t))
    with pytest.raises(ValueError):
        _run(lambda t: ops.subsample(t, (2,)), t)


def test_reductions_histogram_bits():
    x = (rs.rand(4, 6, 3).astype(np.float32) + 0.1)
    _check(_run(lambda x: ops.logsum(x, (0, 2)), x), _torch(lambda x: torch.log(x.sum((0, 2))), x))
    _check(_run(lambda x: ops.logsumexp(x, 1, keepdims=True), x), _torch(lambda x: torch.logsumexp(x, 1, True), x))
    y = rs.randn(4, 5, 3).astype(np.float32)
    _check(_run(lambda x: ops.median(x, 1), y), _torch(lambda x: x.median(1).values, y))
    _check(_run(lambda x: ops.erf(x), y), _torch(torch.erf, y))
    (h,) = _run(lambda x: ops.histogram(x, [-1.0, 0.0, 0.5]), y, grads=False)
    want = [np.sum(y < -1), np.sum((y >= -1) & (y < 0)), np.sum((y >= 0) & (y < 0.5)), np.sum(y >= 0.5)]
    np.testing.assert_array_equal(h, want)
    (h,) = _run(lambda x: ops.histogram(x, [0.5, 1.0], absolute_of_input=True), y, grads=False)
    a = np.abs(y)
    np.testing.assert_array_equal(h, [np.sum(a < 0.5), np.sum((a >= 0.5) & (a < 1)), np.sum(a >= 1)])
    p, q = rs.randint(0, 1 << 20, (7,)).astype(np.int32), rs.randint(0, 1 << 20, (7,)).astype(np.int32)
    for op, ref in ((ops.bitwise_and, np.bitwise_and), (ops.bitwise_or, np.bitwise_or), (ops.bitwise_xor, np.bitwise_xor)):
        (r,) = _run(lambda a, b: op(a, b), p, q, grads=False)
        np.testing.assert_array_equal(r, ref(p, q))
    (r,) = _run(lambda a: ops.bitwise_not(a), p, grads=False)
    np.testing.assert_array_equal(r, ~p)


def test_shaped_dropout_and_normalize_image():
    x = np.ones((8, 16, 4), np.float32)
    seed = np.array([3, 4], np.uint32)
    got = _run(lambda x, s: ops.shaped_dropout(x, s, (8, 1, 4), 0.5), x, seed)
    y, dx = got
    assert set(np.unique(y)) <= {0.0, 2.0} and 0 < (y == 0).mean() < 1
    assert (y == y[:, :1, :]).all()  # whole rows of the middle axis drop together
    np.testing.assert_array_equal(dx, y)
    with pytest.raises(ValueError):
        _run(lambda x, s: ops.shaped_dropout(x, s, (8, 3, 4), 0.5), x, seed)
    img = rs.rand(2, 4, 4, 3).astype(np.float32)
    off, sc = np.array([0.1, 0.2, 0.3], np.float32), np.array([2.0, 3.0, 4.0], np.float32)
    (r,) = _run(lambda i, o, s: ops.normalize_image(i, 0.5, o, s), img, off, sc, grads=False)
    assert r.shape == (2, 4, 4, 4) and (r[..., 3] == 0).all()
    np.testing.assert_allclose(r[..., :3], (img * 0.5 - off) * sc, rtol=1e-6)


def test_extra_var_updates():
    ir = popxl.Ir()
    w0, g0 = rs.randn(6, 4).astype(np.float32), rs.randn(6, 4).astype(np.float32)
    rows = np.array([4, 1, 4], np.int32)
    upd = rs.randn(3, 4).astype(np.float32)
    with ir.main_graph:
        acc = popxl.variable(np.zeros((6, 4), np.float32), name="acc")
        sp = popxl.variable(np.zeros((6, 4), np.float32), name="sp")
        g = popxl.variable(g0, name="g")
        w = popxl.variable(w0, name="w")
        ops.var_updates.accumulate_square_(acc, g, 0.5)
        ops.var_updates.sparse_accumulate_(sp, popxl.constant(upd), popxl.constant(rows), 0, 2.0)
        m = popxl.variable(g0 * 0.1, name="m")
        u = popxl.variable(np.abs(g0), name="u")
        step = popxl.variable(np.array(0.0, np.float32), name="step")
        amax = addons.host_store(ops.var_updates.adamax_updater(m, u, w, step, 0.01, 0.9, 1e-6))
        lamb = addons.host_store(ops.var_updates.lamb_updater(m, acc, w, None, 0.01, None, None, 1e-6))
    with popxl.Session(ir, "cpu") as s:
        out = s.run({})
        np.testing.assert_allclose(s.get_tensor_data(acc), 0.5 * g0 * g0, rtol=1e-6)
        want = np.zeros((6, 4), np.float32)
        np.add.at(want, rows, 2.0 * upd)
        np.testing.assert_allclose(s.get_tensor_data(sp), want, rtol=1e-6)
        assert float(s.get_tensor_data(step)) == 1.0
    np.testing.assert_allclose(out[amax], (g0 * 0.1 / (1 - 0.9)) / (np.abs(g0) + 1e-6) + 0.01 * w0, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(out[lamb], (g0 * 0.1) / (np.sqrt(0.5 * g0 * g0) + 1e-6) + 0.01 * w0, rtol=1e-4, atol=1e-5)


def test_all_reduce_over_device_slots_and_its_gradient_pairings():
    a, b = rs.randn(3, 4).astype(np.float32), rs.randn(3, 4).astype(np.float32)
    wa, wb = rs.randn(3, 4).astype(np.float32), rs.randn(3, 4).astype(np.float32)

    def build(kind):
        def f(x, y, wa_, wb_):
            with popxl.ipu(0):
                x = x * 1.0
            with popxl.ipu(1):
                y = y * 1.0
            ra, rb = kind([x, y], "add", [0, 1])
            return ra * wa_ + rb * wb_

        return f

    C = ops.collectives
    y, da, db, *_ = _run(build(C.all_reduce), a, b, wa, wb)
    np.testing.assert_allclose(y, (a + b) * (wa + wb), rtol=1e-5)
    np.testing.assert_allclose(da, wa + wb, rtol=1e-6)
    np.testing.assert_allclose(db, wa + wb, rtol=1e-6)
    y, da, db, *_ = _run(build(C.all_reduce_identical_grad_inputs), a, b, wa, wb)
    np.testing.assert_allclose(y, (a + b) * (wa + wb), rtol=1e-5)
    np.testing.assert_allclose(da, wa, rtol=1e-6)  # backward identity
    np.testing.assert_allclose(db, wb, rtol=1e-6)
    y, da, db, *_ = _run(build(C.all_reduce_identical_inputs), a, b, wa, wb)
    np.testing.assert_allclose(y, a * wa + b * wb, rtol=1e-5)  # forward identity
    np.testing.assert_allclose(da, wa + wb, rtol=1e-6)
    with pytest.raises(ValueError):
        _run(build(lambda ts, o, ipus: C.all_reduce(ts, o, [0])), a, b, wa, wb)


def test_seed_variable_default_gives_each_replica_its_own_seed():
    ir = popxl.Ir(4)
    with ir.main_graph:
        v, t = addons.seed_variable(11)
        st = addons.host_store(t)
    with popxl.Session(ir, "cpu") as s:
        out = np.asarray(s.run({})[st]).reshape(4, 2)
    assert len({tuple(r) for r in out}) == 4
    np.testing.assert_array_equal(out, popxl.create_seeds(11, replicas=4))
    np.testing.assert_array_equal(popxl.create_seeds(11, replicas=4), popxl.create_seeds(11, replicas=4))
    assert popxl.create_seeds(11, batches_per_step=3, replicas=2).shape == (3, 2, 2)
    from popxl_addons_b200.ops.cross_entropy_sharded_wr_loss import cross_entropy_sharded_wr_loss  # noqa: F401


def test_host_fp8_helpers():
    from popxl_addons_b200.xl.fp8_utils import (host_fp8_mse_scale, host_pow2scale_cast_from_fp8,
                                                host_pow2scale_cast_to_fp8)

    x = np.array([0.0, 0.5, -1.75, 3.0, 100.0, -448.0], np.float32)
    b = host_pow2scale_cast_to_fp8(x, popxl.float8_143, 0)
    assert b.dtype == np.uint8 and b.shape == x.shape
    back = host_pow2scale_cast_from_fp8(b, popxl.float32, 0, popxl.float8_143)
    np.testing.assert_allclose(back, [0.0, 0.5, -1.75, 3.0, 96.0, -448.0])  # 100 rounds to 96 with 3 mantissa bits
    # a power-of-two scale on the way in is undone by its negative on the way out
    b2 = host_pow2scale_cast_to_fp8(x[:4], popxl.float8_152, 3)
    np.testing.assert_allclose(host_pow2scale_cast_from_fp8(b2, popxl.float16, -3, popxl.float8_152), x[:4])
    # overflow: NaN by default, the largest finite value when saturating
    big = np.array([1000.0], np.float32)
    assert np.isnan(host_pow2scale_cast_from_fp8(host_pow2scale_cast_to_fp8(big, popxl.float8_143, 0), popxl.float32, 0))
    sat = host_pow2scale_cast_to_fp8(big, popxl.float8_143, 0, nan_on_overflow=False)
    assert host_pow2scale_cast_from_fp8(sat, popxl.float32, 0)[0] == 448.0
    with pytest.raises(ValueError):
        host_pow2scale_cast_to_fp8(x, popxl.float8_143, 40)
    data = np.random.RandomState(0).uniform(-64, -32, 10).astype(np.float16)
    enc, scale = host_fp8_mse_scale(data, popxl.float8_143)
    assert enc.dtype == np.uint8 and -31 <= scale <= 31
    dec = host_pow2scale_cast_from_fp8(enc, popxl.float32, -scale)
    assert np.abs(dec - data.astype(np.float32)).max() <= np.abs(data).max() * 2.0 ** -3  # within one e4m3 step


def test_tile_and_its_gradient():
    """`tile` with more repeat axes than the operand has dimensions: the gradient sums over the copies (a positional
    table tiled over the sequences of a micro-batch)."""
    x = rs.randn(3, 4).astype(np.float32)
    w = rs.randn(2, 6, 12).astype(np.float32)
    _check(_run(lambda a, b: ops.tile(a, (2, 2, 3)) * b, x, w), _torch(lambda a, b: a.repeat(2, 2, 3) * b, x, w))
    _check(_run(lambda a: ops.tile(a, (5, 1)) * 3.0, x), _torch(lambda a: a.repeat(5, 1) * 3.0, x))
