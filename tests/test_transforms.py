"""Transforms checked the way the reference does it: build the same computation plain and transformed, run both,
compare (tests/integration/test_{gradient_accumulation,recomputation,repeat_graph,batch_serialisation,pipelining}.py
of popxl_addons)."""
from functools import partial

import numpy as np
import pytest

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops
from popxl_addons_b200.layers import Linear
from popxl_addons_b200.patterns import apply_pre_alias_patterns
from popxl_addons_b200.transforms.repeat_graph import repeat_graph
from popxl_addons_b200.transforms.batch_serialisation import (RemoteHandle, batch_serial_buffer, batch_serialise,
                                                             batch_serialise_fwd_and_grad)
from popxl_addons_b200.ops.replicated_all_reduce_TP import (replicated_all_reduce_identical_grad_inputs,
                                                          replicated_all_reduce_identical_inputs)
from popxl_addons_b200.xl.autodiff import ExpectedConnectionType

IO_MODES = ["compute", "io", "io_overlapped"]


class Scale(addons.Module):
    def build(self, x):
        scale = self.add_variable_input("scale", partial(np.full, x.shape, 2.0), x.dtype)
        return x * scale


def _grad_accum_model(with_accumulation):
    np.random.seed(42)
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.random.normal(0, 1, (2, 2)), popxl.float32)
        args, graph = Scale().create_graph(x)
        if with_accumulation:
            dargs, dgraph = addons.autodiff_with_accumulation(graph, [graph.args.scale],
                                                              grads_required=graph.graph.inputs)
        else:
            dgraph = addons.autodiff(graph, grads_required=graph.graph.inputs)
            dargs = addons.NamedVariableFactories()
        scale1, scale2 = args.init(), args.init()
        accum1, accum2 = dargs.init(), dargs.init()
        fwd1, fwd2 = graph.bind(scale1), graph.bind(scale2)
        info1 = fwd1.call_with_info(x)
        info2 = fwd2.call_with_info(*info1.outputs)
        seed = popxl.constant(np.ones((2, 2)), popxl.float32)
        d2 = dgraph.bind(accum1).call(seed, args=dgraph.grad_graph_info.inputs_dict(info2))
        d1 = dgraph.bind(accum2).call(d2[0], args=dgraph.grad_graph_info.inputs_dict(info1))
        streams = [] if with_accumulation else [addons.host_store(t) for t in (d1[1], d2[1])]
    session = popxl.Session(ir, "cpu")
    with session:
        out = session.run()
    if with_accumulation:
        accs = [accum1.accum.scale, accum2.accum.scale]
        res = session.get_tensors_data(accs)
        return tuple(res[t] for t in accs)
    return tuple(out[s] for s in streams)


def test_gradient_accumulation_equals_plain_gradients():
    plain = _grad_accum_model(False)
    acc = _grad_accum_model(True)
    # the accumulators belong to (second layer, first layer); plain outputs are (first, second)
    np.testing.assert_almost_equal(plain[0], acc[1])
    np.testing.assert_almost_equal(plain[1], acc[0])


def test_gradient_accumulation_graph_structure():
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.ones((2, 2)), popxl.float32)
        args, graph = Scale().create_graph(x)
        dargs, dgraph = addons.autodiff_with_accumulation(graph, [graph.args.scale])
        assert sorted(dargs.to_dict().keys()) == ["accum.scale", "mean_accum_counter"]
        n_acc = sum(1 for op in dgraph.graph.ops if op.opdef.name == "accumulate_mean_")
        assert n_acc == 1
        assert len(dgraph.graph.outputs) == 0


def test_running_mean_accumulation_over_calls():
    ir = popxl.Ir()
    data = np.arange(12, dtype=np.float32).reshape(3, 2, 2)
    with ir.main_graph:
        x_stream = popxl.h2d_stream((2, 2), popxl.float32)
        args, graph = Scale().create_graph(x_stream.spec)
        dargs, dgraph = addons.autodiff_with_accumulation(graph, [graph.args.scale])
        w, acc = args.init(), dargs.init()
        for _ in range(3):
            x = ops.host_load(x_stream)
            info = graph.bind(w).call_with_info(x)
            dgraph.bind(acc).call(popxl.constant(np.ones((2, 2)), popxl.float32),
                                  args=dgraph.grad_graph_info.inputs_dict(info))
    ir.num_host_transfers = 3
    s = popxl.Session(ir, "cpu")
    s.run({x_stream: data})
    np.testing.assert_allclose(s.get_tensor_data(acc.accum.scale), data.mean(axis=0), rtol=1e-6)
    assert s.get_tensor_data(acc.mean_accum_counter) == 3


class DoubleLinear(addons.Module):
    def build(self, x):
        y = x + 2
        w1 = self.add_variable_input("w1", partial(np.random.normal, 0, 0.1, (2, 2)), x.dtype)
        w2 = self.add_variable_input("w2", partial(np.random.normal, 0, 0.1, (2, 2)), x.dtype)
        return (y @ w1) @ w2


def _recompute_outputs(recompute):
    np.random.seed(1984)
    ir = popxl.Ir()
    with ir.main_graph:
        x_data, x_h2d, x = addons.host_load(np.random.normal(0, 0.1, (2, 2)).astype(np.float32), popxl.float32, "x")
        args, graph = DoubleLinear().create_graph(x)
        dgraph = addons.autodiff(graph)
        n_graphs = len(ir.graphs)
        if recompute:
            dgraph = addons.recompute_graph(dgraph)
            assert len(ir.graphs) == n_graphs + 1
            kinds = [ec.connection_type for ec in dgraph.grad_graph_info.expected_inputs]
            fwd_ins = [ec.fwd_tensor for ec in dgraph.grad_graph_info.expected_inputs
                       if ec.connection_type == ExpectedConnectionType.Fwd]
            assert all(t in graph.graph.inputs for t in fwd_ins)
        layer = graph.bind(args.init())
        x, *_ = layer.call(x)
        info = layer.call_with_info(x)
        x, *_ = info.outputs
        gradient = popxl.constant(np.ones(x.shape), x.dtype, "gradient")
        outs = dgraph.call(gradient, args=dgraph.grad_graph_info.inputs_dict(info))
        streams = tuple(map(addons.host_store, outs))
    with popxl.Session(ir, "cpu") as session:
        outputs = session.run({x_h2d: x_data})
    return tuple(outputs[s] for s in streams)


def test_recompute_graph_gives_identical_gradients():
    for a, b in zip(_recompute_outputs(False), _recompute_outputs(True)):
        np.testing.assert_almost_equal(a, b)


def test_repeat_graph():
    ir = popxl.Ir()
    with ir.main_graph:
        v = popxl.variable(np.zeros((2,), np.float32), popxl.float32, "v")
        ops.add_(v, popxl.constant(np.ones((2,)), popxl.float32))
        repeat_graph(ir.main_graph, 5)
    s = popxl.Session(ir, "cpu")
    s.run()
    np.testing.assert_array_equal(s.get_tensor_data(v), np.full((2,), 5, np.float32))
    assert len(ir.main_graph.ops) == 1 and ir.main_graph.ops[0].opdef.name == "repeat"


# ---- batch serialisation ---------------------------------------------------------------------------------------


@pytest.mark.parametrize("io_mode", IO_MODES)
def test_batch_serialisation_forward(io_mode):
    bf, cb = 4, 3
    np.random.seed(0)
    inputs = np.random.normal(0, 1, (bf, cb, 8)).astype(np.float32)
    w = np.random.normal(0, 1, (8, 6)).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        in_h2d = popxl.h2d_stream((cb, 8), popxl.float32, "in")
        out_d2h = popxl.d2h_stream((cb, 6), popxl.float32, "out")
        args, graph = Linear(6, bias=False).create_graph(in_h2d.spec)
        result = batch_serialise(graph, bf, {graph.graph.inputs[0]: in_h2d}, {graph.graph.outputs[0]: out_d2h}, {},
                                 io_mode=io_mode)
        weights = args.init()
        result.graph.bind(weights).call(0)
    ir.num_host_transfers = bf
    s = popxl.Session(ir, "cpu")
    s.write_variable_data(weights.weight, w)
    out = s.run({in_h2d: inputs})[out_d2h]
    np.testing.assert_allclose(out, inputs @ w, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("io_mode", IO_MODES)
def test_batch_serialisation_rows_and_offsets(io_mode):
    """Two rows (layers) through one loop graph; input from a remote buffer with row offset, output to another."""
    bf, rows = 3, 2
    np.random.seed(1)
    data = np.random.normal(0, 1, (rows + 1, bf, 2, 4)).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        spec = popxl.TensorSpec((2, 4), popxl.float32)
        args, graph = Scale().create_graph(spec)
        x_in = graph.graph.inputs[0]
        in_buffer = batch_serial_buffer(x_in, steps=bf, rows=rows + 1)
        out_buffer = batch_serial_buffer(graph.graph.outputs[0], steps=bf, rows=rows)
        result = batch_serialise(graph, bf, {x_in: RemoteHandle(in_buffer, 1)}, {},
                                 {graph.graph.outputs[0]: RemoteHandle(out_buffer, 0)}, rows=rows, io_mode=io_mode)
        w = args.init()
        for r in range(rows + 1):
            for i in range(bf):
                ops.remote_store(in_buffer, r * bf + i, popxl.constant(data[r, i]))
        loop = result.graph.bind(w)
        loop.call(0)
        loop.call(1)
        streams = []
        for r in range(rows):
            for i in range(bf):
                streams.append(addons.host_store(ops.remote_load(out_buffer, r * bf + i)))
    assert in_buffer.entries == bf * (rows + 1)
    s = popxl.Session(ir, "cpu")
    out = s.run()
    got = np.stack([out[st] for st in streams]).reshape(rows, bf, 2, 4)
    np.testing.assert_allclose(got, data[1:] * 2.0, rtol=1e-6)


@pytest.mark.parametrize("io_mode", IO_MODES)
def test_batch_serialisation_callable_offset(io_mode):
    bf = 2
    data = np.arange(2 * bf * 4, dtype=np.float32).reshape(2, bf, 4)
    ir = popxl.Ir()
    with ir.main_graph:
        args, graph = Scale().create_graph(popxl.TensorSpec((4,), popxl.float32))
        x_in = graph.graph.inputs[0]
        buf = batch_serial_buffer(x_in, steps=bf, rows=2)
        out_d2h = popxl.d2h_stream((4,), popxl.float32)
        # reads row (1 - n) when called with row n
        res = batch_serialise(graph, bf, {x_in: RemoteHandle(buf, lambda n: popxl.constant(1, popxl.int32) - n)},
                              {graph.graph.outputs[0]: out_d2h}, {}, rows=2, io_mode=io_mode)
        w = args.init()
        for r in range(2):
            for i in range(bf):
                ops.remote_store(buf, r * bf + i, popxl.constant(data[r, i]))
        res.graph.bind(w).call(0)
    ir.num_host_transfers = bf
    s = popxl.Session(ir, "cpu")
    out = s.run()[out_d2h]
    np.testing.assert_allclose(out, data[1] * 2.0)


@pytest.mark.parametrize("io_mode", IO_MODES)
def test_batch_serialised_gradient_equals_plain(io_mode):
    bf, cb = 4, 3
    np.random.seed(7)
    inputs = np.random.normal(0, 1, (bf, cb, 8)).astype(np.float32)
    grads_in = np.random.normal(0, 1, (bf, cb, 6)).astype(np.float32)
    w = np.random.normal(0, 1, (8, 6)).astype(np.float32)

    def plain():
        ir = popxl.Ir()
        with ir.main_graph:
            x = popxl.variable(inputs.reshape(bf * cb, 8), popxl.float32)
            args, graph = Linear(6, bias=False).create_graph(x)
            dgraph = addons.autodiff(graph, grads_required=[graph.args.weight])
            weights = args.init()
            info = graph.bind(weights).call_with_info(x)
            (dw,) = dgraph.call(popxl.constant(grads_in.reshape(bf * cb, 6)),
                                args=dgraph.grad_graph_info.inputs_dict(info))
            st = addons.host_store(dw)
        s = popxl.Session(ir, "cpu")
        s.write_variable_data(weights.weight, w)
        return s.run()[st] / bf

    def serial():
        ir = popxl.Ir()
        with ir.main_graph:
            in_h2d = popxl.h2d_stream((cb, 8), popxl.float32, "in")
            args, graph = Linear(6, bias=False).create_graph(in_h2d.spec)
            dargs, dgraph = addons.autodiff_with_accumulation(graph, [graph.args.weight])
            grad_in = dgraph.graph.inputs[0]
            grad_buffer = batch_serial_buffer(grad_in, steps=bf)
            bs_fwd, bs_grad = batch_serialise_fwd_and_grad(
                graph, dgraph, graph.args, bf,
                load_handles={graph.graph.inputs[0]: in_h2d, grad_in: RemoteHandle(grad_buffer, 0)},
                store_streams={}, store_buffers={}, io_mode=io_mode)
            weights = args.init()
            accs = dargs.init()
            gvars = accs.copy()
            gvars.update(weights)
            for i in range(bf):
                ops.remote_store(grad_buffer, i, popxl.constant(grads_in[i]))
            bs_fwd.graph.bind(weights).call(0)
            bs_grad.graph.bind(gvars).call(0)
        ir.num_host_transfers = bf
        s = popxl.Session(ir, "cpu")
        s.write_variable_data(weights.weight, w)
        s.run({in_h2d: inputs})
        return s.get_tensor_data(accs.accum.weight)

    np.testing.assert_allclose(plain(), serial(), rtol=1e-4, atol=1e-5)


class FeedForwardTP(addons.Module):
    def __init__(self, tp, dp, fc1_size):
        super().__init__()
        self.replica_grouping = popxl.gcg().ir.replica_grouping(stride=tp, group_size=dp)
        self.fc1 = Linear(fc1_size // tp, replica_grouping=self.replica_grouping)

    def build(self, x):
        tp_group = self.replica_grouping.transpose()
        z = replicated_all_reduce_identical_inputs(x, group=tp_group)
        z = ops.gelu(self.fc1(z))
        z = replicated_all_reduce_identical_grad_inputs(z, group=tp_group)
        bias = self.add_variable_input("bias", lambda: np.zeros(z.shape[-1]), z.dtype)
        return ops.gelu(z + bias)


@pytest.mark.parametrize("io_mode", IO_MODES)
def test_batch_serialisation_tp4_dp2_sharded_activations(io_mode):
    cb, bf, tp, dp, shard, in_size = 3, 4, 4, 2, 16, 8
    rf = tp * dp
    np.random.seed(42)
    inputs = np.random.normal(0, 1, (rf, bf, cb, in_size)).astype(np.float32)
    # identical data inside each tensor-parallel group
    inputs = np.repeat(inputs[::tp], tp, axis=0)
    grad_inputs = np.random.normal(0, 1, (bf, cb, shard)).astype(np.float32)
    w = np.random.normal(0, 1, (tp, in_size, shard)).astype(np.float32)
    b = np.ones((tp, shard), np.float32)
    shared_bias = np.full((shard,), 2, np.float32)

    def plain():
        ir = popxl.Ir(replication=rf)
        with ir.main_graph:
            in_h2d = popxl.h2d_stream((bf, cb, in_size), popxl.float32, "in")
            out_d2h = popxl.d2h_stream(in_h2d.shape, in_h2d.dtype, "out")
            args, graph = FeedForwardTP(tp, dp, tp * shard).create_graph(in_h2d.spec)
            dargs, dgraph = addons.autodiff_with_accumulation(graph, graph.args.tensors,
                                                              grads_required=graph.graph.inputs[:1])
            weights = args.init()
            x = ops.host_load(in_h2d)
            info = graph.bind(weights).call_with_info(x)
            (dx,) = dgraph.bind(dargs.init()).call(popxl.constant(grad_inputs),
                                                   args=dgraph.grad_graph_info.inputs_dict(info))
            ops.host_store(out_d2h, dx)
        apply_pre_alias_patterns(ir)
        s = popxl.Session(ir, "cpu")
        s.write_variables_data({weights.fc1.weight: w, weights.fc1.bias: b, weights.bias: shared_bias})
        return s.run({in_h2d: inputs})[out_d2h]

    def serial():
        ir = popxl.Ir(replication=rf)
        tp_group = ir.replica_grouping(stride=1, group_size=tp)
        with ir.main_graph:
            in_h2d = popxl.h2d_stream((cb, in_size), popxl.float32, "in")
            out_d2h = popxl.d2h_stream(in_h2d.shape, in_h2d.dtype, "out")
            args, graph = FeedForwardTP(tp, dp, tp * shard).create_graph(in_h2d.spec)
            dargs, dgraph = addons.autodiff_with_accumulation(graph, graph.args.tensors,
                                                              grads_required=graph.graph.inputs[:1])
            acts = [ec.fwd_tensor for ec in dgraph.grad_graph_info.expected_inputs
                    if ec.connection_type == ExpectedConnectionType.Fwd and ec.fwd_tensor not in graph.args.tensors]
            shardable = [a for a in acts if a.nelms % tp == 0]
            grad_in = dgraph.graph.inputs[0]
            grad_buffer = batch_serial_buffer(grad_in, steps=bf, shard_group=tp_group)
            bs_fwd, bs_grad = batch_serialise_fwd_and_grad(
                graph, dgraph, graph.args, bf,
                load_handles={graph.graph.inputs[0]: in_h2d, grad_in: (grad_buffer, 0, tp_group)},
                store_streams={dgraph.graph.outputs[0]: out_d2h},
                store_buffers={shardable[0]: tp_group}, io_mode=io_mode)
            weights = args.init()
            gvars = dargs.init()
            gvars.update(weights)
            for i in range(bf):
                v = popxl.variable(grad_inputs[i])
                ops.remote_store(grad_buffer, i, ops.collectives.replica_sharded_slice(v, group=tp_group))
            bs_fwd.graph.bind(weights).call(popxl.constant(0))
            bs_grad.graph.bind(gvars).call(popxl.constant(0))
        ir.num_host_transfers = bf
        apply_pre_alias_patterns(ir)
        s = popxl.Session(ir, "cpu")
        s.write_variables_data({weights.fc1.weight: w, weights.fc1.bias: b, weights.bias: shared_bias})
        out = s.run({in_h2d: np.transpose(inputs, (1, 0, 2, 3))})[out_d2h]
        return np.transpose(out, (1, 0, 2, 3))

    np.testing.assert_allclose(plain().reshape(-1), serial().reshape(-1), rtol=1e-4, atol=1e-5)


# ---- pipelining ------------------------------------------------------------------------------------------------


def test_pipeline_two_stage_inference():
    steps = 6
    data = np.random.RandomState(3).normal(0, 1, (steps, 2, 4)).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        with addons.pipelined_execution(steps) as p:
            with p.stage(0), popxl.ipu(0):
                _, x_stream, x = addons.host_load(data[0], popxl.float32, "x")
                x = (x + 1.0).copy_to_ipu(1)
            with p.stage(1), popxl.ipu(1):
                y = x * 3.0
                out = addons.host_store(y)
    ir.num_host_transfers = steps
    s = popxl.Session(ir, "cpu")
    res = s.run({x_stream: data})[out]
    np.testing.assert_allclose(res, (data + 1.0) * 3.0, rtol=1e-6)


def test_pipeline_requires_enough_steps_and_stages():
    ir = popxl.Ir()
    with ir.main_graph:
        with pytest.raises(ValueError, match="at least 2x the number of stages"):
            with addons.pipelined_execution(3) as p:
                with p.stage(0), popxl.ipu(0):
                    _, x_stream, x = addons.host_load(np.zeros((2,), np.float32), popxl.float32, "x")
                    x = x.copy_to_ipu(1)
                with p.stage(1), popxl.ipu(1):
                    addons.host_store(x + 1.0)
    ir = popxl.Ir()
    with ir.main_graph:
        with pytest.raises(RuntimeError, match="must be created in a stage context"):
            with addons.pipelined_execution(4) as p:
                addons.host_load(np.zeros((2,), np.float32), popxl.float32, "x")


def test_pipeline_training_with_stash_equals_sequential():
    steps = 6

    def sequential():
        np.random.seed(42)
        ir = popxl.Ir()
        data = np.random.normal(0, 1, (steps, 1, 4)).astype(np.float32)
        with ir.main_graph:
            _, x_stream, x = addons.host_load(data[0], popxl.float32, "x")
            args, lin = Linear(4).create_graph(x)
            dargs, dlin = addons.autodiff_with_accumulation(lin, [lin.args.weight])
            w, dw = args.init(), dargs.init()
            info = lin.bind(w).call_with_info(x)
            y, *_ = info.outputs
            y = y + 1
            dlin.bind(dw).call(y, args=dlin.grad_graph_info.inputs_dict(info))
        with popxl.Session(ir, "cpu") as s:
            for n in range(steps):
                s.run({x_stream: data[n]})
        return s.get_tensor_data(dw.accum.weight).copy()

    def pipelined():
        np.random.seed(42)
        ir = popxl.Ir()
        data = np.random.normal(0, 1, (steps, 1, 4)).astype(np.float32)
        with ir.main_graph:
            with addons.pipelined_execution(steps) as p:
                with p.stage(0), popxl.ipu(0):
                    _, x_stream, x = addons.host_load(data[0], popxl.float32, "x")
                    args, lin = Linear(4).create_graph(x)
                    dargs, dlin = addons.autodiff_with_accumulation(lin, [lin.args.weight])
                    w, dw = args.init(), dargs.init()
                    info = lin.bind(w).call_with_info(x)
                    y, *_ = info.outputs
                    y = y.copy_to_ipu(1)
                with p.stage(1), popxl.ipu(1):
                    y = y + 1
                    y = y.copy_to_ipu(0)
                with p.stage(2), popxl.ipu(0):
                    dlin.bind(dw).call(y, args=p.stash_and_restore_activations(info, dlin.grad_graph_info))
        ir.num_host_transfers = steps
        with popxl.Session(ir, "cpu") as s:
            s.run({x_stream: data})
        return s.get_tensor_data(dw.accum.weight).copy()

    np.testing.assert_almost_equal(sequential(), pipelined())


# ---- graph passes of the multi-GPU runtime ------------------------------------------------------------------------


def test_matmul_sum_and_collective_fusion_passes_keep_the_numbers():
    """`a1 @ w1 + a2 @ w2` becomes one accumulate-in-epilogue op, `all_reduce(a1 @ w1 + a2 @ w2)` one fused collective
    op; both must give the results (and gradients) of the plain composition."""
    from popxl_addons_b200.parallel import fuse_gemm_collectives, fuse_matmul_sums
    from popxl_addons_b200.testing_utils import ops_of_type

    rs = np.random.RandomState(5)
    a1, a2 = rs.normal(size=(2, 6, 8)).astype(np.float32), rs.normal(size=(2, 6, 4)).astype(np.float32)
    w1, w2 = rs.normal(size=(8, 5)).astype(np.float32), rs.normal(size=(4, 5)).astype(np.float32)

    def run(fuse_ar, fuse_sum):
        ir = popxl.Ir(replication=2)
        with ir.main_graph:
            s1, s2 = popxl.h2d_stream((6, 8), popxl.float32), popxl.h2d_stream((6, 4), popxl.float32)
            x1, x2 = ops.host_load(s1), ops.host_load(s2)
            v1, v2 = popxl.variable(w1, name="w1"), popxl.variable(w2, name="w2")
            y = ops.collectives.replicated_all_reduce(x1 @ v1 + x2 @ v2, "add", ir.replica_grouping())
            z = (x1 @ v1) + (x2 @ v2)
            out_y, out_z = addons.host_store(y), addons.host_store(z)
        n_ar = fuse_gemm_collectives(ir) if fuse_ar else 0
        n_sum = fuse_matmul_sums(ir) if fuse_sum else 0
        names = [op.opdef.name for op in ir.main_graph.ops]
        res = popxl.Session(ir, "cpu").run({s1: a1, s2: a2})
        return res[out_y], res[out_z], n_ar, n_sum, names

    y0, z0, *_ = run(False, False)
    y1, z1, n_ar, n_sum, names = run(True, True)
    assert n_ar == 1 and n_sum == 1 and "matmul2_all_reduce" in names and "matmul_add" in names
    np.testing.assert_allclose(y1, y0, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(z1, z0, rtol=1e-5, atol=1e-5)
    want = (a1 @ w1 + a2 @ w2).sum(axis=0)
    np.testing.assert_allclose(y0[0], want, rtol=1e-5, atol=1e-5)


def test_pruned_recomputation_gives_identical_training_with_less_work():
    """The recomputed forward pass reduced to what the gradient graph reads: same losses and same weights bit for bit
    for every model family (plain, tensor-parallel with and without fused collectives, sequence-parallel, pipelined),
    and the block's output projections, their all-reduce and the residual add are gone from the second pass."""
    import dataclasses
    import os
    import sys

    from popxl_addons_b200.models import decoder as dec
    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_worker import global_tokens

    def run(cfg, prune, **kw):
        dec._SEED[0] = 0
        tr = DecoderTrainer(cfg, micro_batches=2, device="cpu", lr=1e-2, prune_recompute=prune, **kw)
        tr.session.start_profile()
        losses = [tr.step(global_tokens(cfg, 2, seed=s)) for s in range(2)]
        counts = {k: v["count"] for k, v in tr.session.profile_summary().items()}
        weights = {k: np.array(v) for k, v in tr.session.get_named_tensors_data().to_dict().items()}
        names = {g.name: [o.opdef.name for o in g.ops] for g in tr.ir.graphs}
        return losses, weights, counts, names

    cases = [(DecoderConfig.tiny("gptj", dtype="float32", tp=1, dp=1), {}),
             (DecoderConfig.tiny("gptj", dtype="float32", tp=2, dp=1), {}),
             (DecoderConfig.tiny("gptj", dtype="float32", tp=2, dp=2), dict(fused_collectives=False)),
             (DecoderConfig.tiny("llama", dtype="float32", tp=2, dp=1), {}),
             (DecoderConfig.tiny("gpt2", dtype="float32", tp=1, dp=2), {}),
             (dataclasses.replace(DecoderConfig.tiny("gptj", dtype="float32", tp=2, dp=1), sequence_parallel=True), {})]
    for cfg, kw in cases:
        l0, w0, c0, _ = run(cfg, False, **kw)
        l1, w1, c1, names = run(cfg, True, **kw)
        assert l0 == l1, (cfg.family, cfg.tp, cfg.dp)
        assert w0.keys() == w1.keys()
        for k in w0:
            np.testing.assert_array_equal(w0[k], w1[k], err_msg=k)
        gemms = lambda c: sum(v for k, v in c.items() if "matmul" in k or "linear" in k)  # noqa: E731
        assert gemms(c1) < gemms(c0), (cfg.family, cfg.tp, cfg.dp, cfg.sequence_parallel, sorted(c0.items()), sorted(c1.items()))
        if cfg.tp > 1:
            comm = lambda c: sum(v for k, v in c.items() if "all_reduce" in k or "reduce_scatter" in k)  # noqa: E731
            assert comm(c1) < comm(c0), (c0, c1)
        pruned = [n for n in names if "recomp_fwd" in n]
        assert len(pruned) == 1

    # pipelined: the recomputing block graph runs inside the pipeline stages
    import torch

    from popxl_addons_b200.models.pipeline_trainer import PipelineTrainer

    cfg = DecoderConfig.tiny("llama", layers=4, dtype="float32", tp=1, dp=1)
    outs = []
    for prune in (False, True):
        dec._SEED[0] = 0
        tr = PipelineTrainer(cfg, stages=2, micro_batches=6, device="cpu", lr=1e-2, prune_recompute=prune)
        losses = []
        for step in range(2):
            g = torch.Generator().manual_seed(step)
            tok = torch.randint(0, cfg.vocab_size, (6, 1, 1, cfg.seq_len + 1), generator=g, dtype=torch.int32)
            losses.append(np.asarray(tr.session.run({tr.inputs.tokens: tok, tr.inputs.labels: tok})[tr.outputs.loss]))
        outs.append((losses, {k: np.array(v) for k, v in tr.session.get_named_tensors_data().to_dict().items()}))
    for a, b in zip(outs[0][0], outs[1][0]):
        np.testing.assert_array_equal(a, b)
    for k in outs[0][1]:
        np.testing.assert_array_equal(outs[0][1][k], outs[1][1][k], err_msg=k)


def test_prune_graph_keeps_effects_and_drops_pure_calls():
    """`prune_graph`: calls to graphs without effects are dropped when nothing reads them; ops with an effect of their own
    (an in-place update here) stay with everything they depend on; tensors of other graphs are refused."""
    from popxl_addons_b200.transforms.recomputation import prune_graph

    ir = popxl.Ir()

    def inner(a, w):
        return ops.gelu(a @ w)

    def outer(x, w1, w2, counter: popxl.TensorByRef):
        gi = ir.create_graph(inner, x, w1)
        (h,) = ops.call(gi, x, w1)
        (y,) = ops.call(gi, h, w2)
        ops.var_updates.accumulate_(counter, ops.sum(y))  # an effect: stays, and keeps the second call alive
        return x + y, h

    def outer_pure(x, w1, w2):
        gi = ir.create_graph(inner, x, w1)
        (h,) = ops.call(gi, x, w1)
        (y,) = ops.call(gi, h, w2)
        return x + y, h

    rs = np.random.RandomState(0)
    with ir.main_graph:
        x, w1, w2 = (popxl.variable(rs.normal(0, 1, (4, 4)).astype(np.float32), name=n) for n in ("x", "w1", "w2"))
        c1 = popxl.variable(np.zeros((), np.float32), name="c1")
        c2 = popxl.variable(np.zeros((), np.float32), name="c2")
        g = ir.create_graph(outer, x, w1, w2, c1)
        gp = ir.create_graph(outer_pure, x, w1, w2)
        pruned, tmap = prune_graph(g, [g.outputs[1]])
        pruned_pure, _ = prune_graph(gp, [gp.outputs[1]])
        assert [o.opdef.name for o in pruned_pure.ops] == ["call"]
        assert [o.opdef.name for o in pruned.ops] == ["call", "call", "sum", "accumulate_"]
        assert pruned.is_by_ref(pruned.inputs[3]) and len(pruned.outputs) == 1 and tmap[g.inputs[0]] is pruned.inputs[0]
        with pytest.raises(ValueError):
            prune_graph(g, [gp.outputs[1]])
        _, h_full = ops.call(g, x, w1, w2, c1)
        (h_pruned,) = ops.call(pruned, x, w1, w2, c2)
        (h_pure,) = ops.call(pruned_pure, x, w1, w2)
        streams = [addons.host_store(t) for t in (h_full, h_pruned, h_pure)]
    with popxl.Session(ir, "cpu") as s:
        out = s.run()
        np.testing.assert_array_equal(out[streams[0]], out[streams[1]])
        np.testing.assert_array_equal(out[streams[0]], out[streams[2]])
        assert s.get_tensor_data(c1) == s.get_tensor_data(c2) != 0


def test_schedule_collective_overlap_keeps_dependencies_and_update_order():
    """The ops that do not need an all-reduce's result move in front of its consumers; an update of a tensor that a
    consumer reads, and anything behind an op with an unknown effect, stays where it is. Results are unchanged."""
    from popxl_addons_b200.parallel import schedule_collective_overlap

    def build(ir):
        rg = ir.replica_grouping()

        def body(x, w, acc1: popxl.TensorByRef, acc2: popxl.TensorByRef):
            s = ops.collectives.replicated_all_reduce(x, "add", rg)
            y = ops.gelu(s)                                   # consumer of the all-reduce
            ops.var_updates.accumulate_(acc1, y)              # depends on it
            g = x @ w                                         # independent: moves up
            ops.var_updates.accumulate_(acc2, g)              # independent update of another tensor: moves up
            z = y + acc2                                      # reads acc2 after its update: must stay behind it
            ops.var_updates.accumulate_(acc1, g)              # second update of acc1: stays behind the first one
            return z

        with ir.main_graph:
            x = popxl.variable(np.arange(32, dtype=np.float32).reshape(2, 4, 4) / 10, name="x",
                               replica_grouping=ir.replica_grouping(group_size=1))
            w = popxl.variable(np.eye(4, dtype=np.float32) * 2, name="w")
            a1 = popxl.variable(np.zeros((4, 4), np.float32), name="a1")
            a2 = popxl.variable(np.zeros((4, 4), np.float32), name="a2")
            g = ir.create_graph(body, x, w, a1, a2)
            (z,) = ops.call(g, x, w, a1, a2)
            out = addons.host_store(z)
        return g, out, a1, a2

    results = []
    for reorder in (False, True):
        ir = popxl.Ir(replication=2)
        g, out, a1, a2 = build(ir)
        before = [o.opdef.name for o in g.ops]
        assert before == ["all_reduce", "gelu", "accumulate_", "matmul", "accumulate_", "add", "accumulate_"]
        if reorder:
            assert schedule_collective_overlap(ir) == 2
            assert [o.opdef.name for o in g.ops] == ["all_reduce", "matmul", "accumulate_", "gelu", "accumulate_", "add",
                                                     "accumulate_"]
            assert g.ops[2].inputs[0] is g.inputs[3] and g.ops[4].inputs[0] is g.inputs[2] and g.ops[6].inputs[0] is g.inputs[2]
        with popxl.Session(ir, "cpu") as s:
            o = s.run()
            results.append((o[out], s.get_tensor_data(a1), s.get_tensor_data(a2)))
    for a, b in zip(*results):
        np.testing.assert_array_equal(a, b)


def test_schedule_collective_overlap_does_not_reorder_calls_with_transfers():
    """Calls whose graphs store to a host stream, or load from / store to a remote buffer, keep their order: the
    sequence of host items and of buffer accesses is part of the program, whatever the data dependencies say."""
    from popxl_addons_b200.parallel import schedule_collective_overlap

    # two calls that each hold a host_store: the items must come out in program order
    ir = popxl.Ir(replication=2)
    rg = ir.replica_grouping()
    with ir.main_graph:
        x = popxl.variable(np.full((2, 2), 1.0, np.float32), name="x", replica_grouping=ir.replica_grouping(group_size=1))
        w = popxl.variable(np.full((2,), 5.0, np.float32), name="w")
        stream = popxl.d2h_stream((2,), popxl.float32, "out")

        def store(t):
            ops.host_store(stream, t)

        s = ops.collectives.replicated_all_reduce(x, "add", rg)
        y = s + 1
        sg = ir.create_graph(store, y)
        ops.call(sg, y)
        ops.call(sg, w)
    ir.num_host_transfers = 2
    main_before = [o.opdef.name for o in ir.main_graph.ops]
    schedule_collective_overlap(ir)
    assert [o.opdef.name for o in ir.main_graph.ops] == main_before
    with popxl.Session(ir, "cpu") as sess:
        out = sess.run()[stream]
    np.testing.assert_array_equal(np.asarray(out).reshape(2, 2, 2)[:, 0], [[3, 3], [5, 5]])

    # a call that loads from a remote buffer may not jump ahead of the call that stores to it
    ir = popxl.Ir(replication=2)
    rg = ir.replica_grouping()
    with ir.main_graph:
        x = popxl.variable(np.full((2, 2), 1.0, np.float32), name="x", replica_grouping=ir.replica_grouping(group_size=1))
        buf = popxl.remote_buffer((2,), popxl.float32, 1)
        res = popxl.d2h_stream((2,), popxl.float32, "res")

        def put(t):
            ops.remote_store(buf, 0, t)

        def get():
            return ops.remote_load(buf, 0)

        s = ops.collectives.replicated_all_reduce(x, "add", rg)
        y = s * 4
        pg = ir.create_graph(put, y)
        gg = ir.create_graph(get)
        ops.call(pg, y)
        (back,) = ops.call(gg)
        ops.host_store(res, back)
    names = [o.opdef.name for o in ir.main_graph.ops]
    schedule_collective_overlap(ir)
    assert [o.opdef.name for o in ir.main_graph.ops] == names
    with popxl.Session(ir, "cpu") as sess:
        out = sess.run()[res]
    np.testing.assert_array_equal(np.asarray(out).reshape(2, 2)[0], [8, 8])
