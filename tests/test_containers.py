"""DotTree family, streams, array munging, graph cache, input factories (pure host logic)."""
import numpy as np
import pytest

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.dot_tree import DotTree, sanitise
from popxl_addons_b200.array_munging import (handle_negative_axis, pad_axis, repeat, repeat_axis, repeat_shard, shard,
                                             shard2D, squeeze_safe, tensor_parallel_input, tensor_parallel_output,
                                             unshard, unshard2D)
from popxl_addons_b200.xl import ops


def test_dot_tree_insert_get_nested_and_numeric():
    t = DotTree(a=1)
    t.insert("b.c", 2)
    t.insert("b.d.e", 3, overwrite=True)
    assert t.a == 1 and t.b.c == 2 and t["b.d.e"] == 3 and t.get("b").d.e == 3
    with pytest.raises(ValueError, match="already exists"):
        t.insert("a", 5)
    with pytest.raises(ValueError, match="already exists"):
        t.insert("b.f", 5)  # the existing sub-tree is only merged with overwrite=True
    t.insert("a", 5, overwrite=True)
    assert t.a == 5
    with pytest.raises(ValueError, match="not a valid python identifier"):
        t.insert("not valid", 1)
    n = DotTree()
    for i in range(3):
        n.insert(i, i * 10)
    assert n[0] == 0 and n["1"] == 10 and n[-1] == 20 and n[-3] == 0
    with pytest.raises(KeyError, match="Negative numerical key"):
        n[-4]
    with pytest.raises(ValueError, match="cannot be negative"):
        n.insert(-1, 0)
    with pytest.raises(KeyError):
        t.get("missing")
    with pytest.raises(AttributeError, match="No attribute"):
        t.missing
    assert "b.c" in t and "b.zzz" not in t


def test_dot_tree_conversions():
    d = {"x.y": 1, "x.z": 2, "w": 3, "0": 4}
    t = DotTree.from_dict(d)
    assert dict(t.to_dict()) == d
    keys, values = t.unpack()
    assert list(keys) == sorted(d) and list(values) == [d[k] for k in sorted(d)]
    assert dict(DotTree.pack(keys, values).to_dict()) == d
    assert dict(t.map(lambda v: v * 2).to_dict()) == {k: v * 2 for k, v in d.items()}
    f = t.filter_keys(["x.y", "w"])
    assert dict(f.to_dict()) == {"x.y": 1, "w": 3}
    with pytest.raises(ValueError, match="duplicate"):
        t.filter_keys(["w", "w"])
    c = t.copy()
    c.x.insert("new", 9)
    assert "x.new" not in t
    assert t.pop("x.y") == 1 and "x.y" not in t
    other = DotTree.from_dict({"x.z": "Z", "q": "Q"})
    assert t.to_mapping(other) == {2: "Z"}
    sub = t.x
    t._clear()
    assert t.len_flat() == 0 and t.x is sub
    assert sanitise("1a-b.c") == "_1a_b_c"


def test_update_and_len():
    a = DotTree.from_dict({"m.n": 1})
    b = DotTree.from_dict({"m.o": 2, "p": 3})
    with pytest.raises(ValueError, match="already exists"):
        a.update(b)
    a.update(b, overwrite=True)  # a top-level entry of `b` replaces the entry of the same name
    assert dict(a.to_dict()) == {"m.o": 2, "p": 3}
    a.insert("m.n", 1, overwrite=True)  # dotted inserts merge into the existing sub-tree
    assert a.len() == 2 and a.len_flat() == 3 and a.keys() == ["m", "p"] and a.keys_flat() == ["m.o", "m.n", "p"]


@pytest.mark.parametrize("axis", [0, 1, 2, -1])
def test_shard_unshard_round_trip(axis):
    x = np.random.rand(4, 6, 8)
    s = shard(x, 2, axis)
    assert s.shape[0] == 2
    np.testing.assert_array_equal(unshard(s, axis), x)


def test_shard_examples():
    data = np.arange(8).reshape(4, 2)
    np.testing.assert_array_equal(shard(data, 2, 0), [[[0, 1], [2, 3]], [[4, 5], [6, 7]]])
    np.testing.assert_array_equal(shard(data, 2, 1), [[[0], [2], [4], [6]], [[1], [3], [5], [7]]])
    d = np.arange(6).reshape(2, 3)
    np.testing.assert_array_equal(repeat(d, 2, 0), np.stack([d, d]))
    np.testing.assert_array_equal(repeat(d, 2, 1), [[[0, 1, 2], [0, 1, 2]], [[3, 4, 5], [3, 4, 5]]])
    np.testing.assert_array_equal(repeat_axis(d, 2, 0), np.concatenate([d, d]))
    v = np.arange(4)
    np.testing.assert_array_equal(repeat_shard(v, 2, 2, 0, "contiguous"), [[0, 1], [2, 3], [0, 1], [2, 3]])
    np.testing.assert_array_equal(repeat_shard(v, 2, 2, 0, "strided"), [[0, 1], [0, 1], [2, 3], [2, 3]])
    with pytest.raises(ValueError):
        repeat_shard(v, 2, 2, 0, "other")


def test_shard2d_and_helpers():
    x = np.random.rand(10, 3, 4)
    s = shard2D(x, 2, 4, 0, 2)
    assert s.shape == (8, 5, 3, 1)
    np.testing.assert_array_equal(unshard2D(s, 2, 4, 0, 2), x)
    assert pad_axis(np.ones((2, 3)), 5, 1, 7).shape == (2, 5) and pad_axis(np.ones((2, 3)), 5, 1, 7)[0, 4] == 7
    assert squeeze_safe(np.ones((1, 2, 1)), [0, 1, 2]).shape == (2,)
    assert handle_negative_axis(x, -1) == 2
    with pytest.raises(IndexError):
        handle_negative_axis(x, 3)


def test_tensor_parallel_input_output():
    data = np.arange(4 * 3).reshape(4, 3)
    out = tensor_parallel_input(data, tp=2, rf=4)
    assert out.shape == (2, 4, 3)
    np.testing.assert_array_equal(out[0, 0], out[0, 1])
    np.testing.assert_array_equal(out[0, 2], data[1])
    shifted = tensor_parallel_input(data, 2, 4, lambda x, i: x - i * 100)
    np.testing.assert_array_equal(shifted[0, 1], data[0] - 100)
    back = tensor_parallel_output(out, 2, 2, 4, (3,))
    np.testing.assert_array_equal(back, data)
    with pytest.raises(ValueError):
        tensor_parallel_input(data, 3, 4)


def test_streams_containers():
    ir = popxl.Ir()
    with ir.main_graph:
        ins = addons.InputStreams(x=((2, 2), popxl.float32), y=((3,), popxl.int32))
        outs = addons.OutputStreams(z=((1,), popxl.float16))
    assert ins.x.shape == (2, 2) and ins[1].dtype == popxl.int32 and [s.name for s in ins] == ["x", "y"]
    assert len(ins[0:2]) == 2 and outs.z.spec.dtype == popxl.float16
    again = addons.InputStreams.from_streams({"a": ins.x})
    assert again.a is ins.x
    with pytest.raises(AttributeError):
        ins.missing


def test_variable_factory_shapes_and_iterables():
    ir = popxl.Ir(replication=4)
    with ir.main_graph:
        calls = []

        def init():
            calls.append(1)
            return np.ones((2, 3), np.float32) * len(calls)

        t, f = addons.add_variable_input("w", init, popxl.float32)
        assert len(calls) == 1 and f.shape == (2, 3) and t.shape == (2, 3)
        v1 = f.create_tensor("a")
        v2 = f.create_tensor("b")
        it, fi = addons.add_variable_input("it", iter([np.zeros(2, np.float32), np.ones(2, np.float32)]), popxl.float32)
        vi = [fi.create_tensor("i0"), fi.create_tensor("i1")]
        ts, fs = addons.add_replica_sharded_variable_input("s", lambda: np.arange(8, dtype=np.float32), popxl.float32)
        assert fs.shape == (2,) and fs.meta_shape == (8,) and ts.meta_shape == (8,)
        rg = ir.replica_grouping(stride=2, group_size=2)
        tg, fg = addons.add_variable_input("g", lambda: np.zeros(3, np.float32), popxl.float32, replica_grouping=rg)
        vg = fg.create_tensor("g")
        assert vg.shape == (3,) and vg.shape_on_host == (2, 3)
        with pytest.raises(ValueError):
            addons.add_variable_input("bad", np.zeros(3), popxl.float32)
    s = popxl.Session(ir, "cpu")
    assert s.get_tensor_data(v1)[0, 0] == 1 and s.get_tensor_data(v2)[0, 0] == 2
    np.testing.assert_array_equal(s.get_tensor_data(vi[1]), np.ones(2))


def test_graph_cache_and_function_decorator():
    ir = popxl.Ir()

    class Scale(addons.Module):
        def build(self, x):
            return x * self.add_variable_input("s", lambda: np.ones(x.shape, np.float32), popxl.float32)

    with ir.main_graph:
        a = popxl.variable(np.ones((2, 2), np.float32))
        b = popxl.variable(np.ones((2, 2), np.float32))
        c = popxl.variable(np.ones((3,), np.float32))
        m = Scale(cache=True)
        n0 = len(ir.graphs)
        f1, g1 = m.create_graph(a)
        f2, g2 = m.create_graph(b)
        f3, g3 = m.create_graph(c)
        assert g1.graph is g2.graph and g3.graph is not g1.graph and len(ir.graphs) == n0 + 2
        assert f2.to_dict().keys() == f1.to_dict().keys()

        @addons.function
        def twice(x):
            return x + x

        n1 = len(ir.graphs)
        y = twice(a)
        z = twice(b)
        w = twice(c)
        assert len(ir.graphs) == n1 + 2
        st = addons.host_store(z)
    out = popxl.Session(ir, "cpu").run()
    np.testing.assert_array_equal(out[st], np.full((2, 2), 2.0))


def test_streams_from_an_iterable_of_streams():
    ir = popxl.Ir()
    with ir.main_graph:
        a = popxl.h2d_stream((2,), popxl.float32, "a")
        b = popxl.h2d_stream((3,), popxl.int32, "b")
    ins = addons.InputStreams.from_streams([a, b])
    assert list(ins) == [a, b] and ins[0] is a and ins[a.tensor_id] is a and a.tensor_id in ins and len(ins) == 2
    named = addons.InputStreams.from_streams({"x": a})
    assert named.x is a
