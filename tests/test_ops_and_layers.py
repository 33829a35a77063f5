"""Add-on ops and layers against host oracles (torch / numpy / scipy), including the multi-replica ones run on the
in-process replica simulation (the reference's `ir.replication_factor = N` trick)."""
from functools import partial

import numpy as np
import pytest
import torch

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops
from popxl_addons_b200.testing_utils import TensorInput, run_module, ops_of_type


def _run(ir, feeds=None):
    return popxl.Session(ir, "cpu").run(feeds or {})


@pytest.mark.parametrize("stride,size,rf", [(1, 4, 8), (2, 2, 8), (4, 2, 8), (2, 4, 16), (1, 16, 16)])
@pytest.mark.parametrize("op", ["add", "mean"])
def test_strided_collectives(stride, size, rf, op):
    from popxl_addons_b200.ops.replicated_strided_collectives import (replicated_all_gather_strided,
                                                                     replicated_all_reduce_strided,
                                                                     replicated_reduce_scatter_strided)

    np.random.seed(0)
    data = np.random.rand(rf, 2, 6).astype(np.float32)
    ir = popxl.Ir(replication=rf)
    with ir.main_graph:
        h2d = popxl.h2d_stream((2, 6), popxl.float32)
        x = ops.host_load(h2d)
        rg = ir.replica_grouping(stride=stride, group_size=size)
        ar = replicated_all_reduce_strided(x, op, rg)
        rs = replicated_reduce_scatter_strided(x, op, rg)
        ag = replicated_all_gather_strided(rs, rg)
        s_ar, s_rs, s_ag = (addons.host_store(t) for t in (ar, rs, ag))
    out = _run(ir, {h2d: data})
    red = np.add.reduce if op == "add" else np.mean
    n = -(-12 // size)
    for r in range(rf):
        block = r // (stride * size)
        members = [block * stride * size + (r % stride) + j * stride for j in range(size)]
        expect = red(data[members], axis=0)
        np.testing.assert_allclose(out[s_ar][r], expect, rtol=1e-5)
        flat = np.concatenate([expect.reshape(-1), np.zeros(n * size - 12, np.float32)])
        idx = members.index(r)
        np.testing.assert_allclose(out[s_rs][r], flat[idx * n:(idx + 1) * n], rtol=1e-5)
        np.testing.assert_allclose(out[s_ag][r], flat, rtol=1e-5)


def test_two_stage_reduction_equals_one_all_reduce():
    """Reduce-scatter inside a group of consecutive replicas (one node), all-reduce of the shards across the groups,
    all-gather inside the group: the sum over all replicas, with only 1/group_size of the data crossing groups
    (the reference's tests/integration/test_distributed_collectives.py:56-69 builds the same chain)."""
    from popxl_addons_b200.ops.replicated_strided_collectives import (replicated_all_gather_strided,
                                                                     replicated_all_reduce_strided,
                                                                     replicated_reduce_scatter_strided)

    rf, local = 8, 4
    data = np.random.RandomState(5).rand(rf, 5, 7).astype(np.float32)  # 35 elements: not a multiple of the group size
    ir = popxl.Ir(replication=rf)
    with ir.main_graph:
        h2d = popxl.h2d_stream((5, 7), popxl.float32)
        x = ops.host_load(h2d)
        inside = ir.replica_grouping(stride=1, group_size=local)
        across = inside.transpose()
        assert (across.stride, across.group_size) == (local, rf // local)
        shard = replicated_reduce_scatter_strided(x, "add", inside)
        assert shard.shape == (9,)
        shard = replicated_all_reduce_strided(shard, "add", across)
        full = replicated_all_gather_strided(shard, inside)
        st = addons.host_store(ops.reshape(full[:35], (5, 7)))
    out = _run(ir, {h2d: data})
    np.testing.assert_allclose(out[st], np.tile(data.sum(0), (rf, 1, 1)), rtol=1e-5)


def test_tensor_parallel_all_reduce_pairs_and_pattern():
    from popxl_addons_b200.ops.replicated_all_reduce_TP import (replicated_all_reduce_identical_grad_inputs,
                                                              replicated_all_reduce_identical_inputs)
    from popxl_addons_b200.patterns import apply_pre_alias_patterns

    rf = 4
    data = np.random.RandomState(1).rand(rf, 3).astype(np.float32)

    def build(fn):
        ir = popxl.Ir(replication=rf)
        with ir.main_graph:
            h2d = popxl.h2d_stream((3,), popxl.float32)
            x = ops.host_load(h2d)
            g = ir.create_graph(lambda t: fn(t) * 2.0, x)
            dg = popxl.transforms.autodiff(g)
            info = ops.call_with_info(g, x)
            (dx,) = ops.call(dg.graph, popxl.constant(np.ones(3, np.float32)), inputs_dict=dg.inputs_dict(info))
            sy, sd = addons.host_store(info.outputs[0]), addons.host_store(dx)
        return ir, h2d, sy, sd

    ir, h2d, sy, sd = build(lambda t: replicated_all_reduce_identical_inputs(t))
    with pytest.raises(RuntimeError, match="apply_pre_alias_patterns"):
        _run(ir, {h2d: data})
    assert apply_pre_alias_patterns(ir) == 1
    out = _run(ir, {h2d: data})
    np.testing.assert_allclose(out[sy], data * 2)            # forward identity
    np.testing.assert_allclose(out[sd], np.full((rf, 3), 8.0))  # backward all-reduce of 2.0 over 4 replicas
    ir, h2d, sy, sd = build(lambda t: replicated_all_reduce_identical_grad_inputs(t))
    out = _run(ir, {h2d: data})
    np.testing.assert_allclose(out[sy], np.tile(data.sum(0) * 2, (rf, 1)), rtol=1e-6)
    np.testing.assert_allclose(out[sd], np.full((rf, 3), 2.0))


@pytest.mark.parametrize("dtype,decimal", [("float32", 5), ("float16", 2)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy_sharded_vs_torch(dtype, decimal, reduction):
    from popxl_addons_b200.ops.cross_entropy_sharded_loss import cross_entropy_sharded_loss

    tp, n, v = 4, 10, 32
    rng = np.random.RandomState(2)
    logits = rng.randn(n, v).astype(dtype)
    labels = rng.randint(0, v, (n,)).astype(np.int32)
    labels[3] = 5
    ignore = 5
    shard = v // tp
    ir = popxl.Ir(replication=tp)
    xdt = popxl.dtype.as_dtype(dtype)
    with ir.main_graph:
        l_h2d = popxl.h2d_stream((n, shard), xdt)
        i_h2d = popxl.h2d_stream((n,), popxl.int32)
        ig_h2d = popxl.h2d_stream((), popxl.int32)
        lg, idx, ig = ops.host_load(l_h2d), ops.host_load(i_h2d), ops.host_load(ig_h2d)
        g = ir.create_graph(lambda a, b, c: cross_entropy_sharded_loss(a, b, c, reduction=reduction), lg, idx, ig)
        dg = popxl.transforms.autodiff(g, grads_required=[g.inputs[0]])
        info = ops.call_with_info(g, lg, idx, ig)
        loss = info.outputs[0]
        seed = popxl.constant(np.ones(loss.shape, dtype), xdt)
        (dl,) = ops.call(dg.graph, seed, inputs_dict=dg.inputs_dict(info))
        s_loss, s_dl = addons.host_store(loss), addons.host_store(dl)
    feeds = {l_h2d: np.stack(np.split(logits, tp, axis=1)),
             i_h2d: np.stack([labels - r * shard for r in range(tp)]),
             ig_h2d: np.array([ignore - r * shard for r in range(tp)], np.int32)}
    out = _run(ir, feeds)
    tl = torch.tensor(logits.astype(np.float32), requires_grad=True)
    ref = torch.nn.functional.cross_entropy(tl, torch.tensor(labels).long(), ignore_index=ignore, reduction=reduction)
    ref.backward(torch.ones_like(ref))
    for r in range(tp):
        np.testing.assert_almost_equal(out[s_loss][r], ref.detach().numpy(), decimal)
    got = np.concatenate([out[s_dl][r] for r in range(tp)], axis=1)
    np.testing.assert_almost_equal(got, tl.grad.numpy(), decimal)


def test_cross_entropy_sharded_within_replica_uneven():
    from popxl_addons_b200.ops.cross_entropy_sharded_loss import cross_entropy_sharded_wr_loss

    n, v, splits = 6, 53, [14, 14, 14, 11]
    rng = np.random.RandomState(3)
    logits = rng.randn(n, v).astype(np.float32)
    labels = rng.randint(0, v, (n,)).astype(np.int32)
    ir = popxl.Ir()
    with ir.main_graph:
        parts = np.split(logits, np.cumsum(splits)[:-1], axis=1)
        lts = [popxl.variable(p) for p in parts]
        its = [popxl.variable(labels) for _ in parts]
        g = ir.create_graph(lambda *a: cross_entropy_sharded_wr_loss(list(a[:4]), list(a[4:])), *lts, *its)
        dg = popxl.transforms.autodiff(g, grads_required=g.inputs[:4])
        info = ops.call_with_info(g, *lts, *its)
        dls = ops.call(dg.graph, popxl.constant(np.ones(n, np.float32)), inputs_dict=dg.inputs_dict(info))
        s_loss = addons.host_store(info.outputs[0])
        s_d = [addons.host_store(d) for d in dls]
    out = _run(ir)
    tl = torch.tensor(logits, requires_grad=True)
    ref = torch.nn.functional.cross_entropy(tl, torch.tensor(labels).long(), reduction="none")
    ref.sum().backward()
    np.testing.assert_allclose(out[s_loss], ref.detach().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(np.concatenate([out[s] for s in s_d], axis=1), tl.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_layer_norm_distributed_matches_local():
    from popxl_addons_b200.layers.layer_norm_distributed import LayerNormDistributed
    from popxl_addons_b200.layers import LayerNorm

    tp, n, h = 4, 5, 16
    rng = np.random.RandomState(4)
    x = rng.randn(n, h).astype(np.float32)
    w, b = rng.randn(h).astype(np.float32), rng.randn(h).astype(np.float32)
    dy = rng.randn(n, h).astype(np.float32)
    ir = popxl.Ir(replication=tp)
    with ir.main_graph:
        rg = ir.replica_grouping()
        x_h2d, d_h2d = popxl.h2d_stream((n, h // tp), popxl.float32), popxl.h2d_stream((n, h // tp), popxl.float32)
        xt, dt = ops.host_load(x_h2d), ops.host_load(d_h2d)
        facts, graph = LayerNormDistributed(rg).create_graph(xt)
        grad = addons.autodiff(graph)
        v = facts.init()
        info = graph.bind(v).call_with_info(xt)
        dx, dw, db = grad.call(dt, args=grad.grad_graph_info.inputs_dict(info))
        streams = [addons.host_store(t) for t in (info.outputs[0], dx, dw, db)]
    s = popxl.Session(ir, "cpu")
    s.write_variables_data({v.weight: np.stack(np.split(w, tp)), v.bias: np.stack(np.split(b, tp))})
    out = s.run({x_h2d: np.stack(np.split(x, tp, 1)), d_h2d: np.stack(np.split(dy, tp, 1))})
    tx = torch.tensor(x, requires_grad=True)
    tw, tb = torch.tensor(w, requires_grad=True), torch.tensor(b, requires_grad=True)
    ty = torch.nn.functional.layer_norm(tx, (h,), tw, tb, 1e-5)
    ty.backward(torch.tensor(dy))
    cat = lambda st, ax: np.concatenate(list(out[st]), axis=ax)
    np.testing.assert_allclose(cat(streams[0], 1), ty.detach().numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(cat(streams[1], 1), tx.grad.numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(cat(streams[2], 0), tw.grad.numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(cat(streams[3], 0), tb.grad.numpy(), rtol=1e-5, atol=1e-5)


def test_rotary_matches_gptj_formula():
    from popxl_addons_b200.ops.rotary_pos_embed import rotary_pos_embed, trig_tables

    b, h, s, d, rot = 2, 3, 7, 16, 8
    rng = np.random.RandomState(5)
    x = rng.randn(b, s, h, d).astype(np.float32)  # (batch, seq, heads, head_dim), the layout of the reference's op
    sin, cos = trig_tables(s, rot)

    def hf_gptj(x):
        # rotate_every_two formulation of the GPT-J reference implementation
        xr, xp = x[..., :rot], x[..., rot:]
        sin_i = np.repeat(sin, 2, axis=-1)[None, :, None]
        cos_i = np.repeat(cos, 2, axis=-1)[None, :, None]
        x1, x2 = xr[..., ::2], xr[..., 1::2]
        rotated = np.stack((-x2, x1), axis=-1).reshape(xr.shape)
        return np.concatenate([xr * cos_i + rotated * sin_i, xp], axis=-1)

    ir = popxl.Ir()
    with ir.main_graph:
        xv = popxl.variable(x)
        sv, cv = popxl.constant(sin), popxl.constant(cos)  # rank 2 and rank 3 tables are both accepted
        g = ir.create_graph(lambda t, a, c: rotary_pos_embed(t, a, c, rot), xv, sv, cv)
        dg = popxl.transforms.autodiff(g, grads_required=[g.inputs[0]])
        info = ops.call_with_info(g, xv, sv, cv)
        (dx,) = ops.call(dg.graph, info.outputs[0], inputs_dict=dg.inputs_dict(info))
        sy, sd = addons.host_store(info.outputs[0]), addons.host_store(dx)
        with pytest.raises(ValueError, match="rank-4"):
            rotary_pos_embed(popxl.variable(np.zeros((2, 2), np.float32)), sv, cv, rot)
    out = _run(ir)
    np.testing.assert_allclose(out[sy], hf_gptj(x), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(out[sd], x, rtol=1e-5, atol=1e-6)  # the gradient op is the inverse rotation


@pytest.mark.parametrize("dim", [-1, 0])
def test_group_quantize_and_linear_gq(dim):
    from popxl_addons_b200.layers.linear_gq import LinearGQ
    from popxl_addons_b200.ops.group_quantize_decompress import (group_quantize_compress_numpy,
                                                                group_quantize_decompress,
                                                                group_quantize_decompress_numpy)

    rng = np.random.RandomState(6)
    w = rng.randn(128, 64).astype(np.float16)
    packed, scale, bias = group_quantize_compress_numpy(w, 64, dim)
    assert packed.dtype == np.uint16 and packed.shape[-1] == 16
    ref = group_quantize_decompress_numpy(packed, scale, bias, dim)
    assert ref.shape == w.shape and np.abs(ref.astype(np.float32) - w.astype(np.float32)).max() < 0.5
    # first element of a group sits in the most significant nibble
    lo = w.astype(np.float32).reshape(128, 1, 64)[0, 0].min() if dim == -1 else None
    ir = popxl.Ir()
    with ir.main_graph:
        out = group_quantize_decompress(popxl.variable(packed, popxl.uint16), popxl.variable(scale),
                                        popxl.variable(bias), dim=dim)
        st = addons.host_store(out)
    np.testing.assert_allclose(_run(ir)[st].astype(np.float32), ref.astype(np.float32), atol=1e-2)
    lin = torch.nn.Linear(128, 64)
    x = (rng.randn(4, 128) * 0.3).astype(np.float16)
    (y,) = run_module(LinearGQ(64, group_size=64, dim=dim), TensorInput(x, popxl.float16), device="cpu",
                      weights=partial(LinearGQ.torch_mapping, nn_layer=lin, dtype=popxl.float16, group_size=64, dim=dim))
    np.testing.assert_allclose(y.astype(np.float32), lin(torch.tensor(x).float()).detach().numpy(), atol=0.1)


def test_fp8_scales_and_linear_fp8():
    from popxl_addons_b200.layers.linear_fp8 import LinearFP8
    from popxl_addons_b200.ops.fp8_mse_scale import fp8_mse_scale, fp8_mse_scale_reference

    rng = np.random.RandomState(7)
    x = (rng.randn(100) * 3).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        xv = popxl.variable(x)
        s_amax = addons.host_store(addons.fp8_amax_scale(xv, popxl.float8_143))
        s_mse = addons.host_store(fp8_mse_scale(xv, popxl.float8_143))
        s_mse2 = addons.host_store(fp8_mse_scale(xv, popxl.float8_152))
    out = _run(ir)
    assert out[s_amax] == np.clip(np.floor(np.log2(448.0 / np.abs(x).max())), -31, 31)
    assert out[s_amax].dtype == np.int32
    # scaling the data by 2^k moves the best scale by -k
    base = int(fp8_mse_scale_reference(torch.tensor(x), "float8_143", 23))
    assert int(fp8_mse_scale_reference(torch.tensor(x * 16), "float8_143", 23)) == base - 4
    assert int(out[s_mse]) == base and -31 <= int(out[s_mse2]) <= 31
    # data that already fits needs (almost) no scaling; tiny data is scaled up
    assert int(fp8_mse_scale_reference(torch.tensor(x * 2.0 ** -20), "float8_143", 23)) >= base + 19
    lin = torch.nn.Linear(32, 16)
    xin = rng.randn(8, 32).astype(np.float32)
    for metric in ("amax", "mse", "manual_scale"):
        (y,) = run_module(LinearFP8(16, scale_metric=metric, scale=2), TensorInput(xin), device="cpu",
                          weights=lambda v: {v.weight: lin.weight.data.numpy().T.copy(), v.bias: lin.bias.data.numpy()})
        np.testing.assert_allclose(y, lin(torch.tensor(xin)).detach().numpy(), atol=0.1)


def test_linear_fp8_trains():
    """One-layer FP8 classifier trained with hand-written SGD reaches high accuracy on a separable toy problem
    (stands in for the reference's MNIST run, whose data set cannot be downloaded here)."""
    from popxl_addons_b200.layers.linear_fp8 import LinearFP8

    rng = np.random.RandomState(8)
    centers = rng.randn(4, 16).astype(np.float32) * 3
    labels = rng.randint(0, 4, 256)
    xs = centers[labels] + rng.randn(256, 16).astype(np.float32) * 0.3
    ir = popxl.Ir()
    with ir.main_graph:
        x_h2d, l_h2d = popxl.h2d_stream((32, 16), popxl.float32), popxl.h2d_stream((32,), popxl.int32)
        x, lab = ops.host_load(x_h2d), ops.host_load(l_h2d)
        facts, fwd = LinearFP8(4).create_graph(x)
        grad = fwd.autodiff()
        v = facts.init()
        info = fwd.bind(v).call_with_info(x)
        loss, dlogits = addons.cross_entropy_with_grad(info.outputs[0], lab)
        dx, dw, db = grad.call(dlogits, args=grad.grad_graph_info.inputs_dict(info))
        ops.scaled_add_(v.weight, dw, b=-0.05)
        ops.scaled_add_(v.bias, db, b=-0.05)
        s_logits = addons.host_store(info.outputs[0])
    s = popxl.Session(ir, "cpu")
    acc = 0.0
    for epoch in range(6):
        correct = 0
        for i in range(0, 256, 32):
            out = s.run({x_h2d: xs[i:i + 32], l_h2d: labels[i:i + 32].astype(np.int32)})
            correct += (out[s_logits].argmax(-1) == labels[i:i + 32]).sum()
        acc = correct / 256
    assert acc > 0.9


def test_sparse_matmul_grad_square_add_linear_layout():
    from popxl_addons_b200.ops.grad_reduce_square_add import grad_reduce_square_add
    from popxl_addons_b200.ops.linear_layout import linear_layout
    from popxl_addons_b200.ops.static_sparse_ops import dense_const_sparse_matmul, random_sparse

    rng = np.random.RandomState(9)
    lhs = rng.randn(1, 2, 3).astype(np.float32)
    from scipy.sparse import csr_matrix

    dense = rng.randn(3, 4).astype(np.float32)
    np.random.seed(3)
    assert random_sparse(dense, 0.5) is dense and 0 < (dense == 0).sum() < dense.size  # sparsified in place
    csr = csr_matrix(dense)
    g = rng.randn(7, 5).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        s1 = addons.host_store(dense_const_sparse_matmul(popxl.variable(lhs), csr, 4))
        s2 = addons.host_store(grad_reduce_square_add(popxl.variable(g), 64))
        s3 = addons.host_store(ops.sqrt(grad_reduce_square_add(popxl.variable(g), popxl.constant(2.0))))
        s4 = addons.host_store(linear_layout(popxl.variable(g).T, 4))
    out = _run(ir)
    np.testing.assert_allclose(out[s1], lhs @ dense, rtol=1e-5)
    np.testing.assert_allclose(out[s2], ((g / 64) ** 2).sum(), rtol=1e-5)
    np.testing.assert_allclose(out[s3], np.sqrt(((g / 2) ** 2).sum()), rtol=1e-5)
    np.testing.assert_array_equal(out[s4], g.T)


def test_layers_match_torch():
    from popxl_addons_b200.layers import Conv2D, Embedding, GroupNorm, LayerNorm, Linear

    rng = np.random.RandomState(10)
    x = rng.randn(6, 16).astype(np.float32)
    lin = torch.nn.Linear(16, 8)
    (y,) = run_module(Linear(8), TensorInput(x), device="cpu", weights=partial(Linear.torch_mapping, nn_layer=lin))
    np.testing.assert_allclose(y, lin(torch.tensor(x)).detach().numpy(), rtol=1e-3, atol=1e-5)
    ln = torch.nn.LayerNorm(16)
    torch.nn.init.normal_(ln.weight), torch.nn.init.normal_(ln.bias)
    (y,) = run_module(LayerNorm(), TensorInput(x), device="cpu", weights=partial(LayerNorm.torch_mapping, nn_layer=ln))
    np.testing.assert_allclose(y, ln(torch.tensor(x)).detach().numpy(), rtol=1e-3, atol=1e-5)
    with pytest.raises(ValueError, match="2-D"):
        run_module(LayerNorm(), TensorInput(x.reshape(2, 3, 16)), device="cpu")
    img = rng.randn(2, 4, 16, 16).astype(np.float32)
    gn = torch.nn.GroupNorm(2, 4)
    torch.nn.init.normal_(gn.weight), torch.nn.init.normal_(gn.bias)
    (y,) = run_module(GroupNorm(2), TensorInput(img), device="cpu", weights=partial(GroupNorm.torch_mapping, nn_layer=gn))
    np.testing.assert_allclose(y, gn(torch.tensor(img)).detach().numpy(), rtol=1e-3, atol=1e-4)
    for kw, tkw in [(dict(kernel_size=3, paddings=1), dict(padding=1)),
                    (dict(kernel_size=(3, 2), strides=2, dilations=1, groups=2), dict(stride=2, groups=2)),
                    (dict(kernel_size=3, paddings="same_upper"), dict(padding="same"))]:
        conv = torch.nn.Conv2d(4, 6, kw["kernel_size"], **tkw)
        (y,) = run_module(Conv2D(6, **kw), TensorInput(img), device="cpu",
                          weights=partial(Conv2D.torch_mapping, nn_layer=conv))
        np.testing.assert_allclose(y, conv(torch.tensor(img)).detach().numpy(), rtol=1e-3, atol=1e-4)
    emb = torch.nn.Embedding(50, 8)
    idx = rng.randint(0, 50, (5,)).astype(np.int32)
    (y,) = run_module(Embedding(popxl.float32, 50, 8), TensorInput(idx, popxl.int32), device="cpu",
                      weights=partial(Embedding.torch_mapping, nn_layer=emb))
    np.testing.assert_allclose(y, emb(torch.tensor(idx).long()).detach().numpy(), rtol=1e-6)
    assert Embedding.get_vocab_shard_size(50, 4) == 16 and list(Embedding.get_offsets(50, 4)) == [0, 16, 32, 48]
    assert Embedding.get_vocab_shard_size(50, 1) == 64  # padded to a multiple of 16 also when not sharded


def test_sharded_embedding_partial_sums():
    from popxl_addons_b200.layers import Embedding

    tp, vocab, hidden = 4, 50, 8
    emb = torch.nn.Embedding(vocab, hidden)
    idx = np.array([0, 15, 16, 33, 49], np.int32)
    ir = popxl.Ir(replication=tp)
    with ir.main_graph:
        rg = ir.replica_grouping(stride=tp, group_size=1)
        layer = Embedding(popxl.float32, vocab, hidden, replica_grouping=rg)
        i_h2d = popxl.h2d_stream((5,), popxl.int32)
        facts, graph = layer.create_graph(i_h2d.spec)
        v = facts.init()
        (y,) = graph.bind(v).call(ops.host_load(i_h2d))
        y = ops.collectives.replicated_all_reduce(y, "add")
        st = addons.host_store(y)
    s = popxl.Session(ir, "cpu")
    s.write_variables_data(Embedding.torch_mapping(v, emb, tp))
    offsets = Embedding.get_offsets(vocab, tp)
    out = s.run({i_h2d: np.stack([idx - o for o in offsets]).astype(np.int32)})[st]
    for r in range(tp):
        np.testing.assert_allclose(out[r], emb(torch.tensor(idx).long()).detach().numpy(), rtol=1e-6)


def test_adam_module_vs_torch_and_sgd():
    from popxl_addons_b200.optimizers import AdamOptimizerStep, SGDOptimizerStep

    rng = np.random.RandomState(11)
    w0, grads = rng.randn(4, 3).astype(np.float32), [rng.randn(4, 3).astype(np.float32) for _ in range(3)]
    for fused in (True, False):
        ir = popxl.Ir()
        with ir.main_graph:
            w = popxl.variable(w0.copy(), name="w")
            g_h2d = popxl.h2d_stream((4, 3), popxl.float32)
            facts, graph = AdamOptimizerStep(fused=fused).create_graph(w, g_h2d.spec, lr=1e-2, weight_decay=0.0,
                                                                       first_order_dtype=popxl.float32)
            assert sorted(facts.to_dict()) == ["first_order", "second_order", "step"]
            graph.bind(facts.init()).call(w, ops.host_load(g_h2d))
        s = popxl.Session(ir, "cpu")
        tw = torch.tensor(w0.copy(), requires_grad=True)
        opt = torch.optim.AdamW([tw], lr=1e-2, eps=1e-5, weight_decay=0.0)
        for g in grads:
            s.run({g_h2d: g})
            tw.grad = torch.tensor(g)
            opt.step()
        np.testing.assert_almost_equal(s.get_tensor_data(w), tw.detach().numpy(), 4)
    ir = popxl.Ir()
    with ir.main_graph:
        w = popxl.variable(w0.copy(), name="w")
        g_h2d = popxl.h2d_stream((4, 3), popxl.float32)
        facts, graph = SGDOptimizerStep().create_graph(w, g_h2d.spec, lr=0.1, momentum=0.9, weight_decay=0.01)
        graph.bind(facts.init()).call(w, ops.host_load(g_h2d))
    s = popxl.Session(ir, "cpu")
    tw = torch.tensor(w0.copy(), requires_grad=True)
    opt = torch.optim.SGD([tw], lr=0.1, momentum=0.9, weight_decay=0.01)
    for g in grads:
        s.run({g_h2d: g})
        tw.grad = torch.tensor(g)
        opt.step()
    np.testing.assert_allclose(s.get_tensor_data(w), tw.detach().numpy(), rtol=1e-5, atol=1e-6)


def test_cross_entropy_ops_and_misc_utils(capsys):
    rng = np.random.RandomState(12)
    logits = rng.randn(6, 9).astype(np.float32)
    labels = rng.randint(0, 9, (6,)).astype(np.int32)
    ir = popxl.Ir()
    with ir.main_graph:
        lv, tv = popxl.variable(logits), popxl.variable(labels, popxl.int32)
        s_plain = addons.host_store(addons.cross_entropy(lv, tv))
        loss, dl = addons.cross_entropy_with_grad(lv, tv, loss_scaling=4.0)
        s_loss, s_dl = addons.host_store(loss), addons.host_store(dl)
        n_mm = ops_of_type(ir.main_graph.ops, "ce_with_grad")
        flops_before = addons.total_FLOPs(ir)
        y = lv @ popxl.variable(rng.randn(9, 5).astype(np.float32))
        addons.disable_fc_pass(ir)
        addons.set_available_memory_proportion_by_ipu(ir, [0.3])
        table = addons.print_FLOPs(ir)
    assert n_mm == 1 and addons.total_FLOPs(ir) - flops_before == 2 * 9 * 6 * 5 and table["MatMul"] == 540
    breakdown = addons.evaluate_FLOPs(ir.main_graph)
    assert list(breakdown["MatMul"].values()) == [540] and breakdown["TOT"] == addons.total_FLOPs(ir)
    assert ir.options["use_fc_pass"] is False and ir.main_graph.hints["available_memory_proportion"] == {0: 0.3}
    assert addons.format_flops_scientific(2.5e12) == "2.500E+12" and addons.format_flops_scientific(9072) == "9.072E+03"
    assert addons.format_flops_scientific(64, "K") == "0.064E+03"
    out = _run(ir)
    tl = torch.tensor(logits, requires_grad=True)
    ref = torch.nn.functional.cross_entropy(tl, torch.tensor(labels).long())
    (ref * 4.0).backward()
    np.testing.assert_allclose(out[s_plain], ref.item(), rtol=1e-5)
    np.testing.assert_allclose(out[s_loss], ref.item(), rtol=1e-5)
    np.testing.assert_allclose(out[s_dl], tl.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_rts_bucket_step_with_norm_clipping_equals_adam_with_global_norm():
    """Bucketed RTS optimizer with clipping: reduce-scatter of every accumulator + sum of squares of the owned ranges,
    all-reduce of the sums -> global norm -> clip factor, update from the reduced gradients. Must equal the reference's
    composition: gradients averaged over the replicas, `AdamOptimizerStep(global_norm=..., global_norm_max=...)` on
    fp32 weights (popxl_addons/optimizers/adam.py:37-48)."""
    from popxl_addons_b200.optimizers import AdamOptimizerStep
    from popxl_addons_b200.optimizers.rts_adam import rts_adam_bucket_, rts_reduce_bucket_

    dp, max_norm, lr = 2, 0.5, 1e-2
    rng = np.random.RandomState(7)
    shapes = [(8, 6), (16,)]
    w0 = [rng.randn(*s).astype(np.float32) for s in shapes]
    grads = [[rng.randn(*s).astype(np.float32) for s in shapes] for _ in range(dp)]  # per replica
    decays = (0.01, 0.0)

    # reference composition on one replica with the averaged gradients
    mean_g = [np.mean([grads[r][k] for r in range(dp)], axis=0) for k in range(len(shapes))]
    norm = float(np.sqrt(sum((g.astype(np.float64) ** 2).sum() for g in mean_g)))
    ir = popxl.Ir()
    with ir.main_graph:
        gn = popxl.constant(norm, popxl.float32)
        ref_vars = []
        for k, s in enumerate(shapes):
            w = popxl.variable(w0[k], popxl.float32, f"w{k}")
            g = popxl.constant(mean_g[k], popxl.float32)
            facts, graph = AdamOptimizerStep().create_graph(w, g, lr=lr, beta1=0.9, beta2=0.95, eps=1e-5,
                                                            weight_decay=decays[k], first_order_dtype=popxl.float32,
                                                            global_norm=gn, global_norm_max=max_norm)
            graph.bind(facts.init(f"opt{k}")).call(w, g, gn)
            ref_vars.append(w)
    with popxl.Session(ir, "cpu") as s:
        s.run()
        want = [s.get_tensor_data(w).copy() for w in ref_vars]
    assert norm > max_norm  # the clip is active

    # bucketed RTS composition over dp replicas
    ir = popxl.Ir(replication=dp)
    with ir.main_graph:
        rg = ir.replica_grouping()
        one = ir.replica_grouping(group_size=1)
        ws, accs, masters, ms, vs = [], [], [], [], []
        for k, s in enumerate(shapes):
            ws.append(popxl.variable(w0[k].astype(np.float32), popxl.float32, f"w{k}"))
            accs.append(popxl.variable(np.stack([grads[r][k] for r in range(dp)]), popxl.float32, f"acc{k}",
                                       replica_grouping=one))
            master, _ = popxl.replica_sharded_variable(w0[k], popxl.float32, f"master{k}", shard_grouping=rg)
            m, _ = popxl.replica_sharded_variable(np.zeros(s, np.float32), popxl.float32, f"m{k}", shard_grouping=rg)
            v, _ = popxl.replica_sharded_variable(np.zeros(s, np.float32), popxl.float32, f"v{k}", shard_grouping=rg)
            masters.append(master), ms.append(m), vs.append(v)
        step = popxl.variable(np.zeros((), np.float32), popxl.float32, "step")
        sumsq = rts_reduce_bucket_(accs, rg)
        total = ops.collectives.replicated_all_reduce(sumsq, "add", rg)
        gmax = popxl.constant(max_norm, popxl.float32)
        clip = ops.div(gmax, ops.maximum(ops.sqrt(total), gmax))
        rts_adam_bucket_(ws, accs, masters, ms, vs, step, rg, lr=lr, weight_decays=decays, beta1=0.9, beta2=0.95, eps=1e-5,
                         scale=clip, reduced=True)
    with popxl.Session(ir, "cpu") as s:
        s.run()
        for k in range(len(shapes)):
            got = s.get_tensor_data(ws[k])
            np.testing.assert_allclose(got, want[k], rtol=1e-5, atol=1e-6)
        assert float(s.get_tensor_data(step)) == 1.0
