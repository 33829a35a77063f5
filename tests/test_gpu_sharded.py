"""Vocabulary-sharded cross-entropy and hidden-sharded LayerNorm on the device: the same programs run on the CPU backend
(oracle) and on CUDA with all replicas of the group in this process, where every pass over a shard is one of the
package's kernels and only the per-row statistics go through the communicator. The launch counters prove that the
kernels ran and that nothing fell back to the torch implementation."""
import numpy as np
import pytest
import torch

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops

pytestmark = pytest.mark.gpu


@pytest.fixture()
def counters():
    from popxl_addons_b200.ops import native

    native.FALLBACKS.clear()
    before = dict(native.LAUNCHES["by_kernel"])
    strict, native.STRICT[0] = native.STRICT[0], True
    yield lambda: {k: v - before.get(k, 0) for k, v in native.LAUNCHES["by_kernel"].items() if v - before.get(k, 0)}
    native.STRICT[0] = strict


def _both(build, feeds_of, tol):
    """Run `build(ir) -> (streams, feeds builder)` on CPU and CUDA and compare every output."""
    outs = []
    for device in ("cpu", "cuda"):
        ir = popxl.Ir(replication=4)
        streams, handles = build(ir)
        with popxl.Session(ir, device) as s:
            res = s.run(feeds_of(handles))
        outs.append([np.asarray(res[st], dtype=np.float32) for st in streams])
    for a, b in zip(*outs):
        np.testing.assert_allclose(b, a, rtol=tol, atol=tol)
    return outs[1]


@pytest.mark.parametrize("dtype,tol", [(np.float32, 2e-6), (np.float16, 1e-2)])
def test_sharded_cross_entropy_forward_and_autodiff_gradient(counters, dtype, tol):
    from popxl_addons_b200.ops.cross_entropy_sharded_loss import cross_entropy_sharded_loss

    tp, n, v = 4, 96, 4 * 136
    rng = np.random.RandomState(2)
    logits = (rng.randn(n, v) * 2).astype(dtype)
    labels = rng.randint(0, v, (n,)).astype(np.int32)
    shard = v // tp
    xdt = popxl.dtype.as_dtype(dtype)

    def build(ir):
        with ir.main_graph:
            l_h2d = popxl.h2d_stream((n, shard), xdt)
            i_h2d = popxl.h2d_stream((n,), popxl.int32)
            lg, idx = ops.host_load(l_h2d), ops.host_load(i_h2d)
            g = ir.create_graph(lambda a, b: cross_entropy_sharded_loss(a, b, reduction="none"), lg, idx)
            dg = popxl.transforms.autodiff(g, grads_required=[g.inputs[0]])
            info = ops.call_with_info(g, lg, idx)
            seed = popxl.constant(np.full((n,), 0.5, dtype), xdt)
            (dl,) = ops.call(dg.graph, seed, inputs_dict=dg.inputs_dict(info))
            return [addons.host_store(info.outputs[0]), addons.host_store(dl)], (l_h2d, i_h2d)

    feeds = lambda h: {h[0]: np.stack(np.split(logits, tp, axis=1)),  # noqa: E731
                       h[1]: np.stack([labels - r * shard for r in range(tp)])}
    loss, dl = _both(build, feeds, tol)
    ran = counters()
    assert ran.get("ce_shard_stats") == tp and ran.get("ce_shard_nls") == tp and ran.get("ce_nls_grad") == tp, ran
    tl = torch.tensor(logits.astype(np.float32), requires_grad=True)
    ref = torch.nn.functional.cross_entropy(tl, torch.tensor(labels).long(), reduction="none")
    (ref * 0.5).sum().backward()
    np.testing.assert_allclose(loss[0], ref.detach().numpy(), rtol=10 * tol, atol=10 * tol)
    np.testing.assert_allclose(np.concatenate(list(dl), axis=1), tl.grad.numpy(), rtol=10 * tol, atol=10 * tol)


@pytest.mark.parametrize("dtype,tol", [(np.float32, 2e-6), (np.float16, 1e-2)])
def test_sharded_cross_entropy_with_grad_keeps_no_softmax(counters, dtype, tol):
    from popxl_addons_b200.ops.cross_entropy_sharded_loss import cross_entropy_sharded_with_grad

    tp, n, v = 4, 64, 4 * 200
    rng = np.random.RandomState(5)
    logits = (rng.randn(n, v) * 3).astype(dtype)
    labels = rng.randint(0, v, (n,)).astype(np.int32)
    shard = v // tp
    xdt = popxl.dtype.as_dtype(dtype)

    def build(ir):
        with ir.main_graph:
            l_h2d = popxl.h2d_stream((n, shard), xdt)
            i_h2d = popxl.h2d_stream((n,), popxl.int32)
            lg, idx = ops.host_load(l_h2d), ops.host_load(i_h2d)
            loss, dlogits = cross_entropy_sharded_with_grad(lg, idx, 2.0)
            return [addons.host_store(loss), addons.host_store(dlogits)], (l_h2d, i_h2d)

    feeds = lambda h: {h[0]: np.stack(np.split(logits, tp, axis=1)),  # noqa: E731
                       h[1]: np.stack([labels - r * shard for r in range(tp)])}
    loss, dl = _both(build, feeds, tol)
    ran = counters()
    assert ran.get("ce_shard_stats") == tp and ran.get("ce_shard_grad_loss") == tp and "ce_shard_nls" not in ran, ran
    tl = torch.tensor(logits.astype(np.float32), requires_grad=True)
    ref = torch.nn.functional.cross_entropy(tl, torch.tensor(labels).long())
    (ref * 2.0).backward()
    np.testing.assert_allclose(loss[0], float(ref), rtol=10 * tol, atol=10 * tol)
    np.testing.assert_allclose(np.concatenate(list(dl), axis=1), tl.grad.numpy(), rtol=10 * tol, atol=10 * tol)


def test_sharded_cross_entropy_within_replica_uneven_shards(counters):
    from popxl_addons_b200.ops.cross_entropy_sharded_loss import cross_entropy_sharded_wr_loss

    n, v, splits = 40, 530, [144, 136, 140, 110]
    rng = np.random.RandomState(3)
    logits = rng.randn(n, v).astype(np.float32)
    labels = rng.randint(0, v, (n,)).astype(np.int32)
    outs = []
    for device in ("cpu", "cuda"):
        ir = popxl.Ir()
        with ir.main_graph:
            parts = np.split(logits, np.cumsum(splits)[:-1], axis=1)
            lts = [popxl.variable(p) for p in parts]
            its = [popxl.variable(labels) for _ in parts]
            g = ir.create_graph(lambda *a: cross_entropy_sharded_wr_loss(list(a[:4]), list(a[4:])), *lts, *its)
            dg = popxl.transforms.autodiff(g, grads_required=g.inputs[:4])
            info = ops.call_with_info(g, *lts, *its)
            dls = ops.call(dg.graph, popxl.constant(np.ones(n, np.float32)), inputs_dict=dg.inputs_dict(info))
            streams = [addons.host_store(info.outputs[0])] + [addons.host_store(d) for d in dls]
        with popxl.Session(ir, device) as s:
            res = s.run()
        outs.append([res[st] for st in streams])
    ran = counters()
    assert ran.get("ce_shard_stats") == 4 and ran.get("ce_shard_combine") == 1 and ran.get("ce_nls_grad") == 4, ran
    for a, b in zip(*outs):
        np.testing.assert_allclose(b, a, rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.float16, 2e-2)])
def test_distributed_layer_norm_forward_and_all_gradients(counters, dtype, tol):
    from popxl_addons_b200.layers.layer_norm_distributed import LayerNormDistributed

    tp, n, h = 4, 300, 4 * 264
    rng = np.random.RandomState(4)
    x = rng.randn(n, h).astype(dtype)
    w, b = (1 + 0.1 * rng.randn(h)).astype(dtype), (0.1 * rng.randn(h)).astype(dtype)
    dy = rng.randn(n, h).astype(dtype)
    xdt = popxl.dtype.as_dtype(dtype)
    outs = []
    for device in ("cpu", "cuda"):
        ir = popxl.Ir(replication=tp)
        with ir.main_graph:
            rg = ir.replica_grouping()
            x_h2d, d_h2d = popxl.h2d_stream((n, h // tp), xdt), popxl.h2d_stream((n, h // tp), xdt)
            xt, dt = ops.host_load(x_h2d), ops.host_load(d_h2d)
            facts, graph = LayerNormDistributed(rg).create_graph(xt)
            grad = addons.autodiff(graph)
            v = facts.init()
            info = graph.bind(v).call_with_info(xt)
            dx, dw, db = grad.call(dt, args=grad.grad_graph_info.inputs_dict(info))
            streams = [addons.host_store(t) for t in (info.outputs[0], dx, dw, db)]
        with popxl.Session(ir, device) as s:
            s.write_variables_data({v.weight: np.stack(np.split(w, tp)), v.bias: np.stack(np.split(b, tp))})
            res = s.run({x_h2d: np.stack(np.split(x, tp, 1)), d_h2d: np.stack(np.split(dy, tp, 1))})
        outs.append([np.asarray(res[st], dtype=np.float32) for st in streams])
    ran = counters()
    assert ran.get("row_sum_sumsq") == tp and ran.get("ln_apply_stats") == tp, ran
    assert ran.get("ln_shard_bwd_stats") == tp and ran.get("ln_shard_bwd_apply") == tp, ran
    scale = [1, 1, np.sqrt(n), np.sqrt(n)]  # dw / db are sums over the rows
    for a, c, sc in zip(outs[0], outs[1], scale):
        np.testing.assert_allclose(c, a, rtol=tol, atol=tol * sc)
    tx = torch.tensor(x.astype(np.float32), requires_grad=True)
    tw = torch.tensor(w.astype(np.float32), requires_grad=True)
    tb = torch.tensor(b.astype(np.float32), requires_grad=True)
    torch.nn.functional.layer_norm(tx, (h,), tw, tb, 1e-5).backward(torch.tensor(dy.astype(np.float32)))
    cat = lambda t, ax: np.concatenate(list(t), axis=ax)  # noqa: E731
    np.testing.assert_allclose(cat(outs[1][1], 1), tx.grad.numpy(), rtol=10 * tol, atol=10 * tol)
    np.testing.assert_allclose(cat(outs[1][2], 0), tw.grad.numpy(), rtol=10 * tol, atol=10 * tol * np.sqrt(n))
    np.testing.assert_allclose(cat(outs[1][3], 0), tb.grad.numpy(), rtol=10 * tol, atol=10 * tol * np.sqrt(n))
