"""Property-based tests (hypothesis) of the host-side building blocks: containers, array layout helpers, replica
groupings, the strided collectives of the in-process backend, 4-bit group quantisation and FP8 scale selection."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.dot_tree import DotTree
from popxl_addons_b200.xl import ops

FAST = settings(max_examples=40, deadline=None)
SLOW = settings(max_examples=12, deadline=None)

_ident = st.from_regex(r"[a-z][a-z0-9_]{0,5}", fullmatch=True).filter(lambda s: not hasattr(DotTree, s))
_key = st.lists(st.one_of(_ident, st.integers(0, 9).map(str)), min_size=1, max_size=3).map(".".join)


@FAST
@given(st.dictionaries(_key, st.integers(), min_size=1, max_size=8))
def test_dot_tree_round_trip(flat):
    # drop keys that are a prefix of another key (a node cannot be both a leaf and a subtree)
    keys = sorted(flat)
    flat = {k: v for k, v in flat.items() if not any(o != k and o.startswith(k + ".") for o in keys)}
    tree = DotTree.from_dict(flat)
    assert dict(tree.to_dict()) == flat
    assert tree.len_flat() == len(flat)
    names, values = tree.unpack()
    assert list(names) == sorted(names) and dict(zip(names, values)) == flat
    again = DotTree.pack(names, values)
    assert dict(again.to_dict()) == flat
    for k, v in flat.items():
        assert k in tree and tree.get(k) == v
    doubled = tree.map(lambda v: 2 * v)
    assert dict(doubled.to_dict()) == {k: 2 * v for k, v in flat.items()}
    with pytest.raises(ValueError):
        tree.insert(next(iter(flat)), 0)  # duplicates need overwrite=True


@FAST
@given(st.integers(1, 4), st.integers(1, 4), st.integers(1, 3), st.integers(0, 2), st.data())
def test_shard_unshard_and_repeat_shard(n, per, other, axis, data):
    shape = [other, other + 1, other + 2]
    shape[axis] = n * per
    x = np.arange(int(np.prod(shape))).reshape(shape)
    parts = addons.shard(x, n, axis)
    assert parts.shape == (n, *[per if i == axis else s for i, s in enumerate(shape)])
    np.testing.assert_array_equal(addons.unshard(parts, axis), x)
    np.testing.assert_array_equal(addons.unshard_arrays([p[None] for p in parts], axis), x)
    r = data.draw(st.integers(1, 3))
    for mode in ("contiguous", "strided"):
        rs = addons.repeat_shard(x, r, n, axis, mode)
        assert rs.shape[0] == r * n
        for i in range(r * n):
            shard_idx = i % n if mode == "contiguous" else i // r  # s0 s1 s0 s1 against s0 s0 s1 s1
            np.testing.assert_array_equal(rs[i], parts[shard_idx])
    neg = axis - x.ndim
    np.testing.assert_array_equal(addons.shard(x, n, neg), parts)


@FAST
@given(st.sampled_from([1, 2, 3, 4, 6, 8, 12, 16]), st.data())
def test_replica_grouping_partitions_and_transpose(rf, data):
    divisors = [d for d in range(1, rf + 1) if rf % d == 0]
    stride = data.draw(st.sampled_from(divisors))
    size = data.draw(st.sampled_from([d for d in divisors if rf % (stride * d) == 0]))
    ir = popxl.Ir(rf)
    rg = ir.replica_grouping(stride=stride, group_size=size)
    assert rg.group_size == size and rg.num_groups == rf // size
    groups = [list(g) for g in rg.groups]
    assert sorted(r for g in groups for r in g) == list(range(rf))  # a partition of the replicas
    for g in groups:
        assert len(g) == size and all(b - a == stride for a, b in zip(g, g[1:]))
        block = g[0] // (stride * size)
        assert all(r // (stride * size) == block and r % stride == g[0] % stride for r in g)
    assign = rg.assignment
    assert all(assign[r] == gi for gi, g in enumerate(groups) for r in g)
    tr = rg.transpose()
    assert tr.group_size == rg.num_groups and tr.num_groups == size
    # every transposed group picks exactly one member of each group
    for tg in tr.groups:
        assert sorted(assign[r] for r in tg) == list(range(rg.num_groups))
    assert tr.transpose() == rg


@SLOW
@given(st.sampled_from([(4, 1, 4), (4, 2, 2), (8, 2, 2), (8, 1, 2), (8, 4, 2), (6, 3, 2), (6, 1, 3)]),
       st.sampled_from(["add", "mean"]), st.integers(1, 7))
def test_strided_collectives_match_numpy(cfg, op, nelms):
    from popxl_addons_b200.ops.replicated_strided_collectives import (replicated_all_gather_strided,
                                                                     replicated_all_reduce_strided,
                                                                     replicated_reduce_scatter_strided)

    rf, stride, size = cfg
    data = np.random.RandomState(nelms).rand(rf, nelms).astype(np.float32)
    ir = popxl.Ir(rf)
    with ir.main_graph:
        h = popxl.h2d_stream((nelms,), popxl.float32)
        x = ops.host_load(h)
        rg = ir.replica_grouping(stride=stride, group_size=size)
        s_ar = addons.host_store(replicated_all_reduce_strided(x, op, rg))
        rs = replicated_reduce_scatter_strided(x, op, rg)
        s_rs = addons.host_store(rs)
        s_ag = addons.host_store(replicated_all_gather_strided(rs, rg))
    with popxl.Session(ir, "cpu") as s:
        out = s.run({h: data})
    red = np.sum if op == "add" else np.mean
    n = -(-nelms // size)
    for r in range(rf):
        block = r // (stride * size)
        members = [block * stride * size + r % stride + j * stride for j in range(size)]
        want = red(data[members], axis=0)
        np.testing.assert_allclose(out[s_ar][r], want, rtol=1e-5)
        flat = np.concatenate([want, np.zeros(n * size - nelms, np.float32)])
        i = members.index(r)
        np.testing.assert_allclose(out[s_rs][r], flat[i * n:(i + 1) * n], rtol=1e-5)
        np.testing.assert_allclose(out[s_ag][r], flat, rtol=1e-5)


@FAST
@given(st.integers(1, 4), st.integers(1, 3), st.sampled_from([4, 8, 64]), st.sampled_from([-1, 0]), st.integers(0, 1000))
def test_group_quantisation_error_is_at_most_half_a_step(rows, groups, gs, dim, seed):
    from popxl_addons_b200.ops.group_quantize_decompress import (group_quantize_compress_numpy,
                                                                group_quantize_decompress_numpy)

    x = np.random.RandomState(seed).randn(rows, groups * gs).astype(np.float32)
    if dim == 0:
        x = np.ascontiguousarray(x.T)
    packed, scale, bias = group_quantize_compress_numpy(x, gs, dim)
    assert packed.dtype == np.uint16 and packed.shape == (rows, groups, gs // 4) and scale.shape == (rows, groups, 1)
    back = group_quantize_decompress_numpy(packed, scale, bias, dim)
    assert back.shape == x.shape
    step = np.repeat(scale[..., 0], gs, axis=-1)
    step = step if dim == -1 else step.T
    # half a quantisation step, plus the float16 rounding of the group's scale and bias
    assert np.all(np.abs(back.astype(np.float32) - x) <= 0.5 * step.astype(np.float32) + 4e-3 * (1 + np.abs(x)))
    # the extremes of every group are reproduced exactly (codes 0 and 15)
    g = (x if dim == -1 else x.T).reshape(rows, groups, gs)
    b = (back if dim == -1 else back.T).reshape(rows, groups, gs)
    np.testing.assert_allclose(b.min(-1), g.min(-1), rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(b.max(-1), g.max(-1), rtol=4e-3, atol=4e-3)


@FAST
@given(st.floats(1e-6, 1e6), st.sampled_from(["float8_143", "float8_152"]), st.integers(0, 100))
def test_fp8_amax_scale_uses_the_top_octave_without_overflow(magnitude, fmt, seed):
    from popxl_addons_b200.ops.fp8_utils import FP8_FORMATS

    data = (np.random.RandomState(seed).rand(16).astype(np.float32) - 0.5) * np.float32(magnitude)
    ir = popxl.Ir()
    with ir.main_graph:
        sc = addons.host_store(addons.fp8_amax_scale(popxl.variable(data), getattr(popxl, fmt)))
    with popxl.Session(ir, "cpu") as s:
        scale = int(s.run({})[sc])
    assert -31 <= scale <= 31
    amax, fmax = float(np.abs(data).max()), FP8_FORMATS[fmt]["max"]
    if -31 < scale < 31:
        assert amax * 2.0 ** scale <= fmax * (1 + 1e-6)      # no overflow after scaling
        assert amax * 2.0 ** (scale + 1) > fmax * (1 - 1e-6)  # and one more octave would overflow


@SLOW
@given(st.integers(2, 5), st.integers(0, 3), st.integers(0, 100), st.booleans())
def test_pipelined_chain_equals_sequential_chain(n_stages, extra_steps, seed, with_stash):
    """A chain of `n_stages` affine stages on as many device slots, with an optional skip connection from the first
    stage to the last through a stash, pipelined over `2 * n_stages + extra` micro-batches: same outputs as applying
    the stages one after the other."""
    steps = 2 * n_stages + extra_steps
    rs = np.random.RandomState(seed)
    data = rs.normal(0, 1, (steps, 3)).astype(np.float32)
    scales, shifts = rs.uniform(0.5, 1.5, n_stages).astype(np.float32), rs.normal(0, 1, n_stages).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        with addons.pipelined_execution(steps) as p:
            with p.stage(0), popxl.ipu(0):
                _, x_stream, x = addons.host_load(data[0], popxl.float32, "x")
                first = x
                x = (x * float(scales[0]) + float(shifts[0])).copy_to_ipu(1)
            for s in range(1, n_stages):
                with p.stage(s), popxl.ipu(s):
                    x = x * float(scales[s]) + float(shifts[s])
                    if s < n_stages - 1:
                        x = x.copy_to_ipu(s + 1)
                    else:
                        if with_stash:
                            # the first stage's input, kept in a ring buffer until this micro-batch reaches the last stage
                            x = x + p.stash_and_restore_tensor(first, from_stage=0)
                        out = addons.host_store(x)
    ir.num_host_transfers = steps
    with popxl.Session(ir, "cpu") as sess:
        got = sess.run({x_stream: data})[out]
    want = data.copy()
    for s in range(n_stages):
        want = want * scales[s] + shifts[s]
    if with_stash:
        want = want + data
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


@SLOW
@given(st.integers(1, 4), st.integers(1, 3), st.integers(0, 2), st.sampled_from(["compute", "io", "io_overlapped"]),
       st.integers(0, 50))
def test_batch_serialised_rows_equal_the_plain_computation(steps, rows, offset, io_mode, seed):
    """`rows` layers x `steps` micro-batches through one serialised loop graph, input rows read from a remote buffer at
    a row offset, outputs written to another buffer: every entry equals the plain computation on that entry."""
    from functools import partial

    from popxl_addons_b200.transforms.batch_serialisation import RemoteHandle, batch_serial_buffer, batch_serialise

    class Affine(addons.Module):
        def build(self, x):
            w = self.add_variable_input("w", partial(np.full, x.shape, 3.0, np.float32), x.dtype)
            return x * w + 1.0

    data = np.random.RandomState(seed).normal(0, 1, (rows + offset, steps, 2, 3)).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        facts, graph = Affine().create_graph(popxl.TensorSpec((2, 3), popxl.float32))
        x_in, y_out = graph.graph.inputs[0], graph.graph.outputs[0]
        in_buffer = batch_serial_buffer(x_in, steps=steps, rows=rows + offset)
        out_buffer = batch_serial_buffer(y_out, steps=steps, rows=rows)
        result = batch_serialise(graph, steps, {x_in: RemoteHandle(in_buffer, offset)}, {},
                                 {y_out: RemoteHandle(out_buffer, 0)}, rows=rows, io_mode=io_mode)
        w = facts.init()
        for r in range(rows + offset):
            for i in range(steps):
                ops.remote_store(in_buffer, r * steps + i, popxl.constant(data[r, i]))
        loop = result.graph.bind(w)
        for r in range(rows):
            loop.call(r)
        streams = [addons.host_store(ops.remote_load(out_buffer, r * steps + i)) for r in range(rows) for i in range(steps)]
    assert in_buffer.entries == steps * (rows + offset) and out_buffer.entries == steps * rows
    with popxl.Session(ir, "cpu") as s:
        out = s.run()
    got = np.stack([out[st] for st in streams]).reshape(rows, steps, 2, 3)
    np.testing.assert_allclose(got, data[offset:] * 3.0 + 1.0, rtol=1e-6)


_UNARY = {
    "exp": (lambda t: ops.exp(t * 0.3), lambda t: torch.exp(t * 0.3)),
    "tanh": (ops.tanh, torch.tanh),
    "sigmoid": (ops.sigmoid, torch.sigmoid),
    "gelu": (ops.gelu, lambda t: torch.nn.functional.gelu(t)),
    "relu": (ops.relu, torch.relu),
    "swish": (ops.swish, torch.nn.functional.silu),
    "sin": (ops.sin, torch.sin),
    "cos": (ops.cos, torch.cos),
    "negate": (ops.negate, torch.neg),
    "abs": (ops.abs, torch.abs),
    "sqrt": (lambda t: ops.sqrt(ops.abs(t) + 1.0), lambda t: torch.sqrt(t.abs() + 1.0)),
    "log": (lambda t: ops.log(ops.abs(t) + 1.0), lambda t: torch.log(t.abs() + 1.0)),
    "softmax": (lambda t: ops.softmax(t, axis=-1), lambda t: torch.softmax(t, -1)),
    "transpose": (lambda t: ops.transpose(ops.transpose(t) * 2.0), lambda t: (t.t() * 2.0).t()),
    "reshape": (lambda t: ops.reshape(ops.reshape(t, (4, 3)) + 1.0, (3, 4)), lambda t: (t.reshape(4, 3) + 1.0).reshape(3, 4)),
    "slice_concat": (lambda t: ops.concat([t[:, 2:], t[:, :2] * 3.0], axis=1), lambda t: torch.cat([t[:, 2:], t[:, :2] * 3.0], 1)),
    "mean_center": (lambda t: t - ops.mean(t, axis=1, keepdims=True) if hasattr(ops.mean, "__call__") else t,
                    lambda t: t - t.mean(1, keepdim=True)),
    "sum_rows": (lambda t: t + ops.sum(t, axis=0, keepdims=True) * 0.1, lambda t: t + t.sum(0, keepdim=True) * 0.1),
    "self_matmul": (lambda t: (t @ ops.transpose(t)) @ t * 0.1, lambda t: (t @ t.t()) @ t * 0.1),
    "clip": (lambda t: ops.clip(t, -0.5, 0.5), lambda t: t.clamp(-0.5, 0.5)),
    "cumsum": (lambda t: ops.cumsum(t, dim=1) * 0.5, lambda t: torch.cumsum(t, 1) * 0.5),
}
_BINARY = {
    "add": (lambda a, b: a + b, lambda a, b: a + b),
    "sub": (lambda a, b: a - b, lambda a, b: a - b),
    "mul": (lambda a, b: a * b, lambda a, b: a * b),
    "div": (lambda a, b: a / (ops.abs(b) + 1.0), lambda a, b: a / (b.abs() + 1.0)),
    "maximum": (ops.maximum, torch.maximum),
    "minimum": (ops.minimum, torch.minimum),
    "row_broadcast": (lambda a, b: a * b[0:1, :], lambda a, b: a * b[0:1, :]),
    "where": (lambda a, b: ops.where(ops.greater(a, b), a, b * 2.0), lambda a, b: torch.where(a > b, a, b * 2.0)),
}


@settings(max_examples=40, deadline=None)
@given(st.lists(st.one_of(st.tuples(st.just("u"), st.sampled_from(sorted(_UNARY)), st.integers(0, 9)),
                          st.tuples(st.just("b"), st.sampled_from(sorted(_BINARY)), st.integers(0, 9), st.integers(0, 9))),
                min_size=1, max_size=7), st.integers(0, 1000))
def test_autodiff_of_random_programs_matches_torch_autograd(program, seed):
    """Random programs over the differentiable ops: the values and the gradients from the graph autodiff equal those of
    torch.autograd on the same expression (every intermediate value is a candidate operand of later ops, and the result
    sums all of them so that every op's vjp rule takes part)."""
    rs = np.random.RandomState(seed)
    a0, b0 = rs.normal(0, 1, (3, 4)).astype(np.float32), rs.normal(0, 1, (3, 4)).astype(np.float32)

    def run(values, table_index):
        for step in program:
            if step[0] == "u":
                values.append(_UNARY[step[1]][table_index](values[step[2] % len(values)]))
            else:
                values.append(_BINARY[step[1]][table_index](values[step[2] % len(values)], values[step[3] % len(values)]))
        total = values[0]
        for v in values[1:]:
            total = total + v
        return total

    ta, tb = torch.tensor(a0, requires_grad=True), torch.tensor(b0, requires_grad=True)
    ty = run([ta, tb], 1)
    ga, gb = torch.autograd.grad(ty.sum(), (ta, tb), allow_unused=True)
    ir = popxl.Ir()
    with ir.main_graph:
        xa, xb = popxl.variable(a0, name="a"), popxl.variable(b0, name="b")
        g = ir.create_graph(lambda a, b: run([a, b], 0), xa, xb)
        info = ops.call_with_info(g, xa, xb)
        dg = popxl.transforms.autodiff(g)
        grads = ops.call(dg.graph, popxl.constant(np.ones((3, 4), np.float32)), inputs_dict=dg.inputs_dict(info))
        grads = grads if isinstance(grads, (tuple, list)) else (grads,)
        sy = addons.host_store(info.outputs[0])
        sg = [addons.host_store(t) for t in grads]
    with popxl.Session(ir, "cpu") as s:
        out = s.run()
    np.testing.assert_allclose(out[sy], ty.detach().numpy(), rtol=1e-4, atol=1e-5)
    by_input = dict(zip([ec.fwd_tensor for ec in dg.expected_outputs], sg))
    for gin, want in zip(g.inputs, (ga, gb)):
        want = np.zeros((3, 4), np.float32) if want is None else want.numpy()
        assert gin in by_input
        np.testing.assert_allclose(out[by_input[gin]], want, rtol=1e-3, atol=1e-4)


@settings(max_examples=25, deadline=None)
@given(st.lists(st.one_of(st.tuples(st.just("u"), st.sampled_from(sorted(_UNARY)), st.integers(0, 9)),
                          st.tuples(st.just("b"), st.sampled_from(sorted(_BINARY)), st.integers(0, 9), st.integers(0, 9))),
                min_size=1, max_size=6), st.integers(0, 1000), st.integers(1, 3), st.booleans())
def test_recomputation_and_accumulation_of_random_programs(program, seed, calls, prune):
    """For a random program with one parameter: the recomputing gradient graph (which only takes the forward inputs; with
    `prune` its second forward pass is cut down to what the gradient graph reads) gives the gradients of the plain one,
    and the accumulating gradient graph leaves the mean of the per-call gradients."""
    from functools import partial

    rs = np.random.RandomState(seed)
    w0 = rs.normal(0, 1, (3, 4)).astype(np.float32)
    xs = rs.normal(0, 1, (calls, 3, 4)).astype(np.float32)

    class Net(addons.Module):
        def build(self, x):
            values = [x, self.add_variable_input("w", partial(np.copy, w0), x.dtype)]
            for step in program:
                if step[0] == "u":
                    values.append(_UNARY[step[1]][0](values[step[2] % len(values)]))
                else:
                    values.append(_BINARY[step[1]][0](values[step[2] % len(values)], values[step[3] % len(values)]))
            total = values[0]
            for v in values[1:]:
                total = total + v
            return total

    ir = popxl.Ir()
    with ir.main_graph:
        x0 = popxl.variable(xs[0])
        facts, graph = Net().create_graph(x0)
        plain = addons.autodiff(graph)
        facts2, graph2 = Net().create_graph(x0)
        recomputed = addons.recompute_graph(addons.autodiff(graph2), prune_forward=prune)
        if prune:  # the final sum only leads to the output: it is never part of the second pass
            second_pass = recomputed.graph.ops[0].attrs["graph"]
            assert len(second_pass.ops) < len(graph2.graph.ops)
        facts3, graph3 = Net().create_graph(x0)
        acc_facts, accumulating = addons.autodiff_with_accumulation(graph3, [graph3.args.w], grads_required=[])
        w = facts.init()
        acc = acc_facts.init()
        seed_grad = popxl.constant(np.ones((3, 4), np.float32))
        streams = []
        for c in range(calls):
            x = popxl.variable(xs[c], name=f"x{c}")
            i1 = graph.bind(w).call_with_info(x)
            g1 = plain.call(seed_grad, args=plain.grad_graph_info.inputs_dict(i1))
            i2 = graph2.bind(w).call_with_info(x)
            g2 = recomputed.call(seed_grad, args=recomputed.grad_graph_info.inputs_dict(i2))
            i3 = graph3.bind(w).call_with_info(x)
            accumulating.bind(acc).call(seed_grad, args=accumulating.grad_graph_info.inputs_dict(i3))
            streams.append(([addons.host_store(t) for t in g1], [addons.host_store(t) for t in g2]))
        # which output of the plain gradient graph belongs to the parameter
        w_index = [ec.fwd_tensor for ec in plain.grad_graph_info.expected_outputs].index(graph.args.w)
    with popxl.Session(ir, "cpu") as s:
        out = s.run()
        mean_grad = s.get_tensor_data(acc.accum.w)
    per_call = []
    for a, b in streams:
        assert len(a) == len(b)
        for sa, sb in zip(a, b):
            if prune:
                np.testing.assert_array_equal(out[sb], out[sa])
            np.testing.assert_allclose(out[sb], out[sa], rtol=1e-5, atol=1e-6)
        per_call.append(out[a[w_index]])
    np.testing.assert_allclose(mean_grad, np.mean(per_call, axis=0), rtol=1e-4, atol=1e-5)


@SLOW
@given(st.sampled_from([(4, 1, 4, 1, 2), (4, 1, 4, 1, 4), (8, 1, 8, 1, 2), (8, 2, 4, 2, 2), (8, 2, 4, 2, 4), (8, 1, 4, 1, 2),
                        (8, 1, 8, 2, 2), (4, 1, 2, 1, 2), (8, 4, 2, 4, 2)]),
       st.sampled_from(["add", "mean"]), st.sampled_from([8, 12, 16]), st.integers(0, 100))
def test_rts_reduce_then_gather_over_nested_groups(cfg, op, nelms, seed):
    """Gradient-style reduction over a replica group that leaves every replica with its shard inside a shard group
    (equal to the replica group or a subset of it), then the all-gather over the shard group: every replica ends up
    with the full reduced tensor of its replica group."""
    from popxl_addons_b200.rts import gather_replica_sharded_tensor, reduce_replica_sharded_tensor

    rf, r_stride, r_size, s_stride, s_size = cfg
    data = np.random.RandomState(seed).rand(rf, nelms).astype(np.float32)
    ir = popxl.Ir(rf)
    with ir.main_graph:
        h = popxl.h2d_stream((nelms,), popxl.float32)
        x = ops.host_load(h)
        rg = ir.replica_grouping(stride=r_stride, group_size=r_size)
        sg = ir.replica_grouping(stride=s_stride, group_size=s_size)
        shard = reduce_replica_sharded_tensor(x, op, replica_group=rg, shard_group=sg)
        assert shard.shape == (nelms // s_size,) and tuple(shard.meta_shape) == (nelms,)
        full = gather_replica_sharded_tensor(shard, replica_group=sg)
        s_shard, s_full = addons.host_store(shard), addons.host_store(full)
    with popxl.Session(ir, "cpu") as s:
        out = s.run({h: data})
    red = np.sum if op == "add" else np.mean
    for r in range(rf):
        block = r // (r_stride * r_size)
        members = [block * r_stride * r_size + r % r_stride + j * r_stride for j in range(r_size)]
        want = red(data[members], axis=0)
        sblock = r // (s_stride * s_size)
        smembers = [sblock * s_stride * s_size + r % s_stride + j * s_stride for j in range(s_size)]
        i, n = smembers.index(r), nelms // s_size
        np.testing.assert_allclose(out[s_shard][r], want[i * n:(i + 1) * n], rtol=1e-5)
        np.testing.assert_allclose(out[s_full][r].reshape(-1), want, rtol=1e-5)
