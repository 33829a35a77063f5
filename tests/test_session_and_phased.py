"""TaskSession checkpoints (incl. replica-grouped and replica-sharded variables), memmap-backed variables, seed
variable, remote buffers and phased execution with replicated tensor sharding."""
import json
import os
from functools import partial

import numpy as np
import pytest

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.layers import Linear
from popxl_addons_b200.named_tensors import NamedTensors
from popxl_addons_b200.remote import (load_remote, load_remote_graph, named_buffers, named_variable_buffers,
                                      store_remote, store_remote_graph)
from popxl_addons_b200.rts import (all_gather_replica_sharded_graph, reduce_replica_sharded_graph,
                                   reduce_replica_sharded_tensor, replica_sharded_spec)
from popxl_addons_b200.task_session import TaskSession, initialise_memmap_dir_from_checkpoint
from popxl_addons_b200.xl import ops


def _linear_session(memmap_dir=None, rf=1):
    ir = popxl.Ir(replication=rf)
    with ir.main_graph:
        ins = addons.InputStreams(x=((2, 4), popxl.float32))
        outs = addons.OutputStreams(y=((2, 3), popxl.float32))
        x = ops.host_load(ins.x)
        facts, graph = Linear(3).create_graph(x)
        variables = facts.init(memmap_dir=memmap_dir) if memmap_dir else facts.init()
        (y,) = graph.bind(variables).call(x)
        ops.host_store(outs.y, y)
    return TaskSession(ins, outs, variables, 2, ir, "cpu"), variables


def test_checkpoint_layout_rotation_and_missing(tmp_path, caplog):
    s, v = _linear_session()
    x = np.ones((2, 4), np.float32)
    s.run({s.inputs.x: x})
    s.add_session_state_info({"note": "hello"})
    dirs = [str(tmp_path / f"ck{i}") for i in range(3)]
    for d in dirs:
        s.save_checkpoint(d)
    assert not os.path.exists(dirs[0]) and os.path.exists(dirs[1]) and os.path.exists(dirs[2])  # max_checkpoints=2
    assert sorted(os.listdir(os.path.join(dirs[2], "model"))) == ["bias.npz", "weight.npz"]
    info = json.load(open(os.path.join(dirs[2], "session_info.json")))
    assert info == {"steps": 1, "note": "hello"}
    s2, v2 = _linear_session()
    s2.load_checkpoint(dirs[2])
    np.testing.assert_array_equal(s2.get_tensor_data(v2.weight), s.get_tensor_data(v.weight))
    assert s2.session_state["steps"] == 1
    os.remove(os.path.join(dirs[2], "model", "bias.npz"))
    os.remove(os.path.join(dirs[2], "session_info.json"))
    with pytest.raises(ValueError, match="not in the loaded state"):
        s2.load_checkpoint(dirs[2], report_missing="error")
    s2.load_checkpoint(dirs[2], report_missing="warn")
    assert s2.session_state == {"steps": 0}
    s3, _ = _linear_session()
    s3.load_from_session(s)
    np.testing.assert_array_equal(s3.run({s3.inputs.x: x})[s3.outputs.y], s.run({s.inputs.x: x})[s.outputs.y])

    class Loader:
        def save(self, path):
            open(path, "w").write("42")

        def resume(self, path):
            self.state = open(path).read()

    s.dataloader = Loader()
    with pytest.raises(ValueError):
        s.dataloader = object()
    s.save_checkpoint(str(tmp_path / "with_dl"))
    s2.dataloader = Loader()
    s2.load_checkpoint(str(tmp_path / "with_dl"))
    assert s2.dataloader.state == "42"


def test_checkpoint_of_grouped_and_sharded_variables(tmp_path):
    rf = 4
    ir = popxl.Ir(replication=rf)
    full = np.arange(16, dtype=np.float32).reshape(2, 8)
    with ir.main_graph:
        tp_rg = ir.replica_grouping(stride=2, group_size=2)  # 2 groups
        grouped = popxl.variable(np.stack([full[0], full[1]]), popxl.float32, "grouped", replica_grouping=tp_rg)
        sharded, _ = popxl.replica_sharded_variable(full[0], popxl.float32, "sharded")
        state = NamedTensors(grouped=grouped, sharded=sharded)
        ops.add_(sharded, popxl.constant(np.ones(2, np.float32)))
    s = TaskSession(addons.InputStreams(), addons.OutputStreams(), state, 1, ir, "cpu")
    assert sharded.shape == (2,) and sharded.meta_shape == (8,) and grouped.shape_on_host == (2, 8)
    s.run()
    s.save_checkpoint(str(tmp_path / "ck"))
    with np.load(tmp_path / "ck" / "model" / "sharded.npz") as z:
        np.testing.assert_array_equal(z["sharded"], full[0] + 1)  # saved unsharded, in its full shape
    with np.load(tmp_path / "ck" / "model" / "grouped.npz") as z:
        assert z["grouped"].shape == (2, 8)
    s.write_variable_data(sharded, np.zeros(8, np.float32))
    s.load_checkpoint(str(tmp_path / "ck"))
    np.testing.assert_array_equal(s.get_tensor_data(sharded), full[0] + 1)


def test_memmap_backed_variables(tmp_path):
    mm = str(tmp_path / "mm")
    np.random.seed(0)
    s, v = _linear_session(memmap_dir=mm)
    assert sorted(os.listdir(mm)) == ["bias.npy", "weight.npy"]
    w = s.get_tensor_data(v.weight)
    # raw arrays without a header: the layout the reference's `np.memmap` files have
    np.testing.assert_array_equal(np.fromfile(os.path.join(mm, "weight.npy"), np.float32).reshape(w.shape), w)
    assert w is v.weight._memmap_arr and isinstance(w, np.memmap)
    s2, v2 = _linear_session(memmap_dir=mm)  # existing files are re-opened, not re-initialised
    np.testing.assert_array_equal(s2.get_tensor_data(v2.weight), w)
    s.save_checkpoint(str(tmp_path / "ck"))
    assert sorted(os.listdir(tmp_path / "ck" / "model")) == ["bias.npy", "weight.npy"]
    initialise_memmap_dir_from_checkpoint(str(tmp_path / "ck"), str(tmp_path / "mm2"))
    s3, v3 = _linear_session(memmap_dir=str(tmp_path / "mm2"))
    np.testing.assert_array_equal(s3.get_tensor_data(v3.weight), w)
    s3.load_checkpoint(str(tmp_path / "ck"))
    np.testing.assert_array_equal(s3.get_tensor_data(v3.weight), w)
    # files with a numpy header are accepted too, and a file of the wrong size is refused
    mm3 = tmp_path / "mm3"
    mm3.mkdir()
    np.save(mm3 / "weight.npy", np.asarray(w))
    np.save(mm3 / "bias.npy", np.asarray(s.get_tensor_data(v.bias)))
    s4, v4 = _linear_session(memmap_dir=str(mm3))
    np.testing.assert_array_equal(s4.get_tensor_data(v4.weight), w)
    np.asarray(w).ravel()[:-1].tofile(mm3 / "weight.npy")
    with pytest.raises(ValueError, match="expected"):
        _linear_session(memmap_dir=str(mm3))


def test_seed_variable_identical_within_group_and_checkpointed():
    ir = popxl.Ir(replication=4)
    with ir.main_graph:
        rg = ir.replica_grouping(stride=1, group_size=2)
        var, seed = addons.seed_variable(7, rg)
        st = addons.host_store(seed)
        a, b = ops.split_random_seed(seed)
        sa, sb = addons.host_store(a), addons.host_store(b)
        d = addons.host_store(ops.dropout(popxl.constant(np.ones(64, np.float32)), a, 0.5))
    s = popxl.Session(ir, "cpu")
    out = s.run()
    seeds = out[st]
    np.testing.assert_array_equal(seeds[0], seeds[1])
    np.testing.assert_array_equal(seeds[2], seeds[3])
    assert not np.array_equal(seeds[0], seeds[2]) and s.get_tensor_data(var).shape == (2, 2)
    assert not np.array_equal(out[sa][0], out[sb][0])
    np.testing.assert_array_equal(out[d][0], out[d][1])  # same seed, same mask
    assert 10 < (out[d][0] == 0).sum() < 54


def test_remote_buffers_load_store_graphs():
    ir = popxl.Ir()
    data = np.arange(24, dtype=np.float32).reshape(3, 2, 4)
    with ir.main_graph:
        facts, graph = Linear(4, bias=False).create_graph(popxl.TensorSpec((2, 2), popxl.float32))
        buffers = named_variable_buffers(facts, entries=3, shard_over_dict=False)
        layers = [facts.init_remote(buffers, i, f"layer{i}") for i in range(3)]
        load, names = load_remote_graph(buffers, entries=3)
        store = store_remote_graph(buffers, entries=3)
        streams = []
        for i in range(3):
            loaded = NamedTensors.pack(names, load.call(i))
            streams.append(addons.host_store(loaded.weight))
            store.bind(NamedTensors(weight=loaded.weight + 100.0)).call(i)
        again = load_remote(buffers, 1)
        st_again = addons.host_store(again.weight)
        store_remote(buffers, NamedTensors(weight=again.weight * 0.0), 2)
        nb = named_buffers(NamedTensors(t=again.weight), entries=2)
        assert nb.t.entries == 2 and nb.t.tensor_shape == (2, 4)
    s = popxl.Session(ir, "cpu")
    for i, lv in enumerate(layers):
        s.write_variable_data(lv.weight, data[i])
    out = s.run()
    for i in range(3):
        np.testing.assert_array_equal(out[streams[i]], data[i])
    np.testing.assert_array_equal(out[st_again], data[1] + 100)
    np.testing.assert_array_equal(s.get_tensor_data(layers[0].weight), data[0] + 100)
    np.testing.assert_array_equal(s.get_tensor_data(layers[2].weight), np.zeros((2, 4)))
    with pytest.raises(RuntimeError, match="remote variable"):
        ir2 = popxl.Ir()
        with ir2.main_graph:
            rb = popxl.remote_buffer((2,), popxl.float32, 1)
            rv = popxl.remote_variable(np.zeros(2, np.float32), rb)
            addons.host_store(rv + 1.0)
        popxl.Session(ir2, "cpu").run()


def test_phased_execution_with_rts():
    """Per layer: load weight shards from their remote buffer, all-gather, compute, reduce-scatter the gradient over
    the data-parallel group, SGD on the shard, store the shard back."""
    rf, n_layers = 4, 2
    np.random.seed(1)
    w0 = np.random.rand(n_layers, 4, 4).astype(np.float32)
    xs = np.random.rand(rf, 2, 4).astype(np.float32)
    ir = popxl.Ir(replication=rf)
    with ir.main_graph:
        dp = ir.replica_grouping()
        x_h2d = popxl.h2d_stream((2, 4), popxl.float32)
        x = ops.host_load(x_h2d)
        facts, fwd = Linear(4, bias=False).create_graph(x)
        grad = addons.autodiff(fwd, grads_required=[fwd.args.weight, fwd.graph.inputs[0]])
        buffers = named_variable_buffers(facts, entries=n_layers)  # sharded over the whole DP group
        assert buffers.weight.meta_shape == (4, 4) and buffers.weight.tensor_shape == (4,)
        layer_vars = [facts.init_remote(buffers, i, f"l{i}") for i in range(n_layers)]
        load, names = load_remote_graph(buffers, n_layers)
        store = store_remote_graph(buffers, n_layers)
        shard_spec = NamedTensors.pack(names, load.graph.outputs)
        gather, gnames = all_gather_replica_sharded_graph(shard_spec)
        reduce, rnames = reduce_replica_sharded_graph(NamedTensors(weight=fwd.args.weight), "mean",
                                                      replica_group=dp)
        acts, infos, shards = x, [], []
        for i in range(n_layers):
            w_shard = NamedTensors.pack(names, load.call(i))
            w_full = NamedTensors.pack(gnames, gather.bind(w_shard).call())
            info = fwd.bind(w_full).call_with_info(acts)
            infos.append((info, w_shard))
            acts = info.outputs[0]
        dy = acts * 0.0 + 1.0
        for i in reversed(range(n_layers)):
            info, w_shard = infos[i]
            dw, dy = grad.call(dy, args=grad.grad_graph_info.inputs_dict(info))
            g_shard = NamedTensors.pack(rnames, reduce.bind(NamedTensors(weight=dw)).call())
            assert g_shard.weight.shape == (4,) and g_shard.weight.meta_shape == (4, 4)
            new = ops.scaled_add(w_shard.weight, g_shard.weight, b=-0.1)
            store.bind(NamedTensors(weight=new)).call(i)
        st = addons.host_store(acts)
    s = popxl.Session(ir, "cpu")
    for i, lv in enumerate(layer_vars):
        s.write_variable_data(lv.weight, w0[i])
    out = s.run({x_h2d: xs})[st]
    np.testing.assert_allclose(out, xs @ w0[0] @ w0[1], rtol=1e-5)
    # closed form of the data-parallel mean gradients
    h1 = xs @ w0[0]
    g1 = np.mean([h1[r].T @ np.ones((2, 4), np.float32) for r in range(rf)], axis=0)
    g0 = np.mean([xs[r].T @ (np.ones((2, 4), np.float32) @ w0[1].T) for r in range(rf)], axis=0)
    np.testing.assert_allclose(s.get_tensor_data(layer_vars[1].weight), w0[1] - 0.1 * g1, rtol=1e-5)
    np.testing.assert_allclose(s.get_tensor_data(layer_vars[0].weight), w0[0] - 0.1 * g0, rtol=1e-5)


def test_tensor_parallel_with_rts_subgroup():
    """rf=8, TP2: the RTS group is a sub-group (stride 2, size 2) of the DP group (stride 2, size 4): all-reduce over
    the DP group followed by a local slice."""
    rf, tp = 8, 2
    ir = popxl.Ir(replication=rf)
    data = np.random.RandomState(2).rand(rf, 8).astype(np.float32)
    with ir.main_graph:
        dp = ir.replica_grouping(stride=tp, group_size=rf // tp)
        rts = ir.replica_grouping(stride=tp, group_size=2)
        h2d = popxl.h2d_stream((8,), popxl.float32)
        x = ops.host_load(h2d)
        spec = replica_sharded_spec(x, rts)
        assert spec.shape == (4,) and spec.meta_shape == (8,)
        assert replica_sharded_spec(popxl.constant(np.zeros(7, np.float32)), rts).shape == (7,)
        red = reduce_replica_sharded_tensor(x, "add", replica_group=dp, shard_group=rts)
        same = reduce_replica_sharded_tensor(x, "add", replica_group=rts, shard_group=rts)
        odd = reduce_replica_sharded_tensor(popxl.variable(np.ones(7, np.float32)), "add", replica_group=rts)
        s1, s2, s3 = addons.host_store(red), addons.host_store(same), addons.host_store(odd)
    out = popxl.Session(ir, "cpu").run({h2d: data})
    for r in range(rf):
        dp_members = [m for m in range(rf) if m % tp == r % tp]
        total = data[dp_members].sum(0)
        idx = rts.index_in_group(r)
        np.testing.assert_allclose(out[s1][r], total[idx * 4:(idx + 1) * 4], rtol=1e-5)
        pair = data[rts.group_of(r)].sum(0)
        np.testing.assert_allclose(out[s2][r], pair[idx * 4:(idx + 1) * 4], rtol=1e-5)
        np.testing.assert_allclose(out[s3][r], np.full(7, 2.0))


def test_named_replica_grouping_helpers(monkeypatch):
    from popxl_addons_b200.named_replica_grouping import (NamedReplicaGrouping, get_ild_replica_grouping,
                                                         get_instance_replica_grouping, is_cross_ild,
                                                         is_cross_instance)

    ir = popxl.Ir(replication=16)
    with ir.main_graph:
        tp = ir.replica_grouping(stride=1, group_size=4)
        dp = ir.replica_grouping(stride=4, group_size=4)
        assert tp.transpose() == dp and dp.transpose() == tp and tp != dp
        named = NamedReplicaGrouping.build_groups(["a", "b.c"], tp)
        assert named.b.c is tp
        assert not is_cross_instance(tp)  # single process hosts all replicas
        assert get_instance_replica_grouping(dp) == dp
        assert not is_cross_ild(tp) and is_cross_ild(dp)  # default NVSwitch domain: 8 ranks
        assert get_ild_replica_grouping(tp).num_replicas == 8
        monkeypatch.setenv("XL_NVLINK_DOMAIN_SIZE", "16")
        assert not is_cross_ild(dp)
        groups = ir.replica_grouping(stride=2, group_size=2)
        assert groups.groups[0] == [0, 2] and groups.groups[1] == [1, 3] and groups.groups[2] == [4, 6]
        assert groups.index_in_group(6) == 1 and groups.num_groups == 8
        with pytest.raises(ValueError):
            ir.replica_grouping(stride=3, group_size=4)


def test_options_and_per_op_profile(monkeypatch):
    """Typed options with environment overrides; the per-op profile counts and times what ran."""
    monkeypatch.setenv("XL_CUDA_GRAPHS", "0")
    monkeypatch.setenv("XL_COLLECTIVE_TIMEOUT_S", "42")
    o = popxl.Options.from_env()
    assert o.cuda_graphs is False and o.collective_timeout_s == 42.0 and o.native_kernels is True
    o["some_planner_hint"] = 0.3  # unknown names are kept as hints
    assert o["some_planner_hint"] == 0.3 and "some_planner_hint" in o and o.get("other", 7) == 7
    ir = popxl.Ir()
    ir.options.profile_ops = True
    with ir.main_graph:
        x = popxl.variable(np.ones((4, 4), np.float32), name="x")
        g = ir.create_empty_graph("body")
        with g:
            a = popxl.graph_input((4, 4), popxl.float32, "a", by_ref=True)
            ops.var_updates.copy_var_update_(a, ops.gelu(a @ a))
        ops.repeat(g, 3, inputs_dict={a: x})
    s = popxl.Session(ir, "cpu")
    s.run({})
    summary = s.profile_summary()
    assert summary["matmul"]["count"] == 3 and summary["gelu"]["count"] == 3 and summary["matmul"]["ms"] >= 0.0
    assert "repeat" not in summary and s.profile is None


def test_run_to_run_determinism_check():
    """The bitwise repeat-run comparison passes for an ordinary training step and reports a program whose result
    depends on something outside its inputs and state."""
    from popxl_addons_b200.debugging import check_run_to_run_determinism
    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer

    cfg = DecoderConfig.tiny("gptj", dtype="float32", tp=2, dp=1)
    tr = DecoderTrainer(cfg, micro_batches=2, device="cpu", lr=1e-2)
    tok = tr.synthetic_tokens(seed=0, pinned=False)
    assert check_run_to_run_determinism(tr.session, {tr.inputs.tokens: tok}) == []
    # a program that draws fresh random numbers each run is reported
    ir = popxl.Ir()
    with ir.main_graph:
        seed = popxl.variable(np.array([1, 2], np.uint32), popxl.uint32, name="seed")
        acc = popxl.variable(np.zeros(4, np.float32), name="acc")
        noise = ops.random_normal(seed, (4,))
        ops.var_updates.accumulate_(acc, noise)
        new_seed, _ = ops.split_random_seed(seed)
        out = addons.host_store(noise)
    s = popxl.Session(ir, "cpu")
    assert check_run_to_run_determinism(s, {}) == []  # same seed variable restored before each run -> same numbers
    import torch

    calls = {"n": 0}
    from popxl_addons_b200.xl.opdef import OPS

    orig = OPS["random_normal"].impl

    def unseeded(*a, **k):
        calls["n"] += 1
        r = orig(*a, **k)
        return r + calls["n"] if r.device.type != "meta" else r

    OPS["random_normal"].impl = unseeded
    try:
        assert "acc" in " ".join(check_run_to_run_determinism(s, {}))
    finally:
        OPS["random_normal"].impl = orig


def test_bump_allocator_canaries_name_the_overrun_allocation():
    import torch
    from popxl_addons_b200.parallel.symm import BumpAllocator

    plain = BumpAllocator(torch.zeros(1 << 16, dtype=torch.uint8), start=1024)
    a = plain.alloc((100,), torch.float32)
    b = plain.alloc((3, 5), torch.bfloat16)
    assert b.data_ptr() - a.data_ptr() == 512  # 400 bytes round up to 512
    plain.check_guards()
    guarded = BumpAllocator(torch.zeros(1 << 16, dtype=torch.uint8), start=1024, guards=True)
    a = guarded.alloc((100,), torch.float32)
    b = guarded.alloc((3, 5), torch.bfloat16)
    assert b.data_ptr() - a.data_ptr() == 512 + 256
    a.fill_(1.0)
    b.fill_(2.0)
    guarded.check_guards()
    # a write that runs 8 bytes over the end of `b`
    flat = guarded.buf[b.data_ptr() - guarded.buf.data_ptr():][:30 + 8]
    flat.fill_(0)
    with pytest.raises(RuntimeError, match=r"allocation #1 .*8 guard bytes changed"):
        guarded.check_guards()
    with pytest.raises(MemoryError):
        guarded.alloc((1 << 16,), torch.uint8)


def test_session_host_interface_and_recorded_options():
    """`expected_inputs`, `create_host_outputs`, `run_with_outputs`, and the IPU session options that programs set
    through `ir._pb_ir.getSessionOptions()` (recorded, without effect)."""
    ir = popxl.Ir(2)
    opts = ir._pb_ir.getSessionOptions()
    opts.numIOTiles = 64
    opts.engineOptions["debug.allowOutOfMemory"] = "true"
    opts.replicatedCollectivesSettings.prepareScheduleForMergingCollectives = True
    assert opts.numIOTiles == 64 and opts.engineOptions["debug.allowOutOfMemory"] == "true"
    with ir.main_graph:
        h = popxl.h2d_stream((3,), popxl.float32, "x")
        x = ops.host_load(h)
        d = popxl.d2h_stream((3,), popxl.float32, "y")
        ops.host_store(d, x * 2.0)
    with popxl.Session(ir, "ipu_model") as s:
        assert s.is_attached and s.expected_inputs() == [h]
        outs = s.create_host_outputs()
        assert {k: v.shape for k, v in outs.items()} == {d: (2, 3)}
        data = np.arange(6, dtype=np.float32).reshape(2, 3)
        s.run_with_outputs({h: data}, outs)
        np.testing.assert_array_equal(outs[d], data * 2)
    assert not s.is_attached


def test_import_aliases_resolve_to_this_package():
    """`import popxl_addons_b200.compat` lets an unedited popxl / popxl_addons program import and run."""
    import subprocess
    import sys
    import textwrap

    prog = textwrap.dedent("""
        import numpy as np
        import popxl_addons_b200.compat
        import popxl, popdist
        from popxl import ops
        import popxl.ops as ops2
        import popxl_addons as addons
        from popxl_addons.layers import Linear
        from popxl.tensor import Variable
        from popxl.utils import to_numpy
        from popxl.ops.call import CallSiteInfo
        from popxl.transforms.autodiff import GradGraphInfo
        from popxl_addons.ops.rotary_pos_embed.rotary_pos_embed import rotary_pos_embed
        from popxl_addons.ops.replicated_strided_collectives.replicated_all_reduce_strided import (
            replicated_all_reduce_strided)
        from popxl_addons.ops.replicated_strided_collectives import replicated_all_reduce_strided as again
        import popxl_addons_b200
        assert popxl is popxl_addons_b200.xl and addons is popxl_addons_b200 and ops is ops2
        assert callable(ops.call) and callable(again) and again is replicated_all_reduce_strided
        assert callable(addons.transforms.autodiff) and callable(popxl.transforms.autodiff)
        assert not popdist.isPopdistEnvSet() and popdist.getNumInstances() == 1
        ir = popxl.Ir()
        with ir.main_graph:
            x = popxl.variable(np.ones((2, 3), np.float32))
            assert isinstance(x, Variable)
            facts, graph = Linear(4).create_graph(x)
            (y,) = graph.bind(facts.init()).call(x)
            st = addons.host_store(y)
        with popxl.Session(ir, "ipu_model") as session:
            print(session.run()[st].shape)
    """)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=repo)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    res = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.strip().endswith("(2, 4)")


def test_weights_and_biases_paths_with_a_stand_in(tmp_path, monkeypatch):
    """Timer summaries, per-variable histograms with non-finite counts and `wandb://` checkpoints, against a stand-in
    for the optional wandb module that records what it is given."""
    import types

    import popxl_addons_b200.task_session as ts
    import popxl_addons_b200.utils as ut

    logged, artifacts = [], {}

    class Artifact:
        def __init__(self, name, type):
            self.name, self.type, self.dir = name, type, None

        def add_dir(self, d):
            import shutil

            self.dir = str(tmp_path / f"artifact_{self.name}")
            shutil.copytree(d, self.dir)

        def download(self):
            return self.dir

    fake = types.SimpleNamespace(
        run=types.SimpleNamespace(summary={}), Histogram=lambda data: ("hist", len(data)),
        log=lambda d, step=None: logged.append((d, step)), Artifact=Artifact,
        log_artifact=lambda a: artifacts.__setitem__(a.name, a),
        use_artifact=lambda name, type=None: {a.name: a for a in artifacts.values() if a.type == type}[name])
    monkeypatch.setattr(ts, "wandb", fake)
    monkeypatch.setattr(ut, "wandb", fake)
    monkeypatch.setattr(ut, "_HAVE_WANDB", True)
    with addons.timer("Unit Test Phase"):
        pass
    assert "unit_test_phase_mins" in fake.run.summary
    s, v = _linear_session()
    s.write_variable_data(v.bias, np.array([1.0, np.nan, np.inf], np.float32))
    s.wandb_variable_histograms(step=7)
    by_name = {k: (val, step) for d, step in logged for k, val in d.items()}
    # key names of the reference (popxl_addons/task_session.py:115-121)
    assert by_name["bias:histogram"] == (("hist", 1), 7) and by_name["bias:not_finite"] == (2, 7)
    assert by_name["weight:not_finite"][0] == 0
    s.run({s.inputs.x: np.ones((2, 4), np.float32)})
    w = s.get_tensor_data(v.weight).copy()
    s.save_checkpoint("wandb://ckpt")
    assert artifacts["ckpt"].type == "checkpoints"  # what the reference saves and looks up
    assert sorted(os.listdir(os.path.join(artifacts["ckpt"].dir, "model"))) == ["bias.npz", "weight.npz"]
    s2, v2 = _linear_session()
    s2.load_checkpoint("wandb://ckpt")
    np.testing.assert_array_equal(s2.get_tensor_data(v2.weight), w)
    assert s2.session_state["steps"] == 1


@pytest.mark.parametrize("family", ["gpt2", "gptj", "llama"])
def test_trainer_with_several_sequences_per_micro_batch(family):
    """Micro-batches of more than one sequence (the GPT-2-small data-parallel configuration uses 8): the positional
    table is tiled over the sequences and its gradient sums over them; data parallel with sharded optimizer state gives
    the losses of the single replica on the same data."""
    import dataclasses

    from popxl_addons_b200.models.decoder import DecoderConfig
    from popxl_addons_b200.models.trainer import DecoderTrainer

    cfg = DecoderConfig.tiny(family, dtype="float32")
    tr = DecoderTrainer(cfg, micro_batches=2, micro_batch_size=3, device="cpu", lr=1e-2)
    tok = tr.synthetic_tokens(seed=0, pinned=False)
    losses = [tr.step(tok) for _ in range(3)]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]
    tr2 = DecoderTrainer(dataclasses.replace(cfg, dp=2), micro_batches=2, micro_batch_size=3, device="cpu", lr=1e-2)
    tok2 = tr2.synthetic_tokens(seed=0, pinned=False)
    l2 = [tr2.step(tok2) for _ in range(2)]
    assert all(np.isfinite(l2)) and l2[-1] < l2[0]
