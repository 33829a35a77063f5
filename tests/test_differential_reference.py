"""Differential tests against the reference's own pure-Python modules (array layout helpers, DotTree), loaded from the
offline installation under `baseline/_ref` by file path and driven with generated inputs. Skipped where that
installation is absent."""
import importlib.util
import itertools
import os
import sys
import types

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import popxl_addons_b200 as addons
from popxl_addons_b200.dot_tree import DotTree

REF_PKG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "popxl_addons")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(REF_PKG, "array_munging.py")),
                                reason="the reference is not installed under baseline/_ref")
FAST = settings(max_examples=60, deadline=None)


def _load(name):
    """A reference module as `ref_<name>`, with the two third-party helpers it imports provided if missing and
    `popxl` / `popxl_addons.utils` resolved by this package."""
    if "more_itertools" not in sys.modules:
        try:
            import more_itertools  # noqa: F401
        except ImportError:
            m = types.ModuleType("more_itertools")
            m.flatten = itertools.chain.from_iterable
            m.sliced = lambda seq, n: (seq[i:i + n] for i in range(0, len(seq), n))
            m.peekable = None
            sys.modules["more_itertools"] = m
    import popxl_addons_b200.compat  # noqa: F401

    spec = importlib.util.spec_from_file_location(f"ref_{name}", os.path.join(REF_PKG, f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref_am():
    return _load("array_munging")


@pytest.fixture(scope="module")
def ref_dt():
    return _load("dot_tree")


def _same(a, b):
    if isinstance(a, (list, tuple)):
        assert isinstance(b, (list, tuple)) and len(a) == len(b)
        for x, y in zip(a, b):
            _same(x, y)
    else:
        a, b = np.asarray(a), np.asarray(b)
        assert a.shape == b.shape and a.dtype == b.dtype
        np.testing.assert_array_equal(a, b)


@FAST
@given(st.integers(1, 4), st.integers(1, 3), st.integers(1, 3), st.integers(-3, 2), st.integers(1, 3))
def test_shard_family(ref_am, n, per, other, axis, reps):
    shape = [other, other + 1, other + 2]
    shape[axis] = n * per
    x = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    _same(addons.shard(x, n, axis), ref_am.shard(x, n, axis))
    parts = ref_am.shard(x, n, axis)
    _same(addons.unshard(parts, axis), ref_am.unshard(parts, axis))
    _same(addons.unshard_arrays([p[None] for p in parts], axis), ref_am.unshard_arrays([p[None] for p in parts], axis))
    _same(addons.repeat(x, reps, axis % x.ndim), ref_am.repeat(x, reps, axis % x.ndim))
    _same(addons.repeat_axis(x, reps, axis), ref_am.repeat_axis(x, reps, axis))
    _same(addons.repeat_shard(x, reps, n, axis, "contiguous"), ref_am.repeat_shard(x, reps, n, axis, "contiguous"))
    if reps == n or reps == 1 or n == 1:
        _same(addons.repeat_shard(x, reps, n, axis, "strided"), ref_am.repeat_shard(x, reps, n, axis, "strided"))
    else:
        # the reference reshapes the tiled shards to (n_shards, n_repeats) instead of (n_repeats, n_shards) before it
        # swaps the axes (array_munging.py:253), which scrambles the order unless the two counts are equal; here every
        # shard is repeated in place, as its docstring describes
        want = np.repeat(ref_am.shard(x, n, axis), reps, axis=0)
        _same(addons.repeat_shard(x, reps, n, axis, "strided"), want)
    assert addons.handle_negative_axis(x, axis) == ref_am.handle_negative_axis(x, axis)
    _same(addons.pad_axis(x, shape[axis] + reps, axis, 7), ref_am.pad_axis(x, shape[axis] + reps, axis, 7))


@FAST
@given(st.integers(1, 3), st.integers(1, 3), st.integers(1, 3), st.integers(1, 3), st.sampled_from([(0, 1), (1, 0), (0, 2), (2, 1)]))
def test_two_axis_sharding(ref_am, n1, n2, p1, p2, axes):
    a1, a2 = axes
    shape = [2, 3, 4]
    shape[a1], shape[a2] = n1 * p1, n2 * p2
    x = np.arange(int(np.prod(shape))).reshape(shape)
    _same(addons.split2D(x, n1, n2, a1, a2), ref_am.split2D(x, n1, n2, a1, a2))
    s = ref_am.shard2D(x, n1, n2, a1, a2)
    _same(addons.shard2D(x, n1, n2, a1, a2), s)
    _same(addons.unshard2D(s, n1, n2, a1, a2), ref_am.unshard2D(s, n1, n2, a1, a2))
    np.testing.assert_array_equal(addons.unshard2D(s, n1, n2, a1, a2), x)


@FAST
@given(st.sampled_from([(1, 2), (2, 2), (2, 4), (4, 4), (1, 4), (2, 8)]), st.integers(1, 3), st.integers(1, 3))
def test_tensor_parallel_host_layouts(ref_am, tp_rf, transfers, width):
    from popxl_addons_b200.array_munging import tensor_parallel_output

    tp, rf = tp_rf
    dp = rf // tp
    data = np.arange(transfers * dp * width, dtype=np.float32).reshape(transfers * dp, width)
    got, want = addons.tensor_parallel_input(data, tp, rf), ref_am.tensor_parallel_input(data, tp, rf)
    _same(got, want)
    double = lambda a, i: a * (i + 1)  # noqa: E731
    _same(addons.tensor_parallel_input(data, tp, rf, double), ref_am.tensor_parallel_input(data, tp, rf, double))
    out = np.asarray(want).reshape(transfers, rf, width)
    for identical in (True, False):
        for true_n in (None, 1):
            _same(tensor_parallel_output(out, transfers, tp, rf, (width,), identical, true_n),
                  ref_am.tensor_parallel_output(out, transfers, tp, rf, (width,), identical, true_n))
    if tp > 1:
        with pytest.raises(ValueError):
            addons.tensor_parallel_input(data, rf * 2, rf)


@FAST
@given(st.lists(st.integers(1, 3), min_size=1, max_size=4), st.data())
def test_squeeze_safe(ref_am, shape, data):
    x = np.zeros(shape)
    ones = [i for i, s in enumerate(shape) if s == 1]
    axis = data.draw(st.one_of(st.none(), st.sampled_from(ones)) if ones else st.none())
    _same(addons.squeeze_safe(x, axis), ref_am.squeeze_safe(x, axis))


_ident = st.from_regex(r"[a-z][a-z0-9_]{0,4}", fullmatch=True).filter(lambda s: not hasattr(DotTree, s))
_key = st.lists(st.one_of(_ident, st.integers(0, 5).map(str)), min_size=1, max_size=3).map(".".join)


@FAST
@given(st.dictionaries(_key, st.integers(), min_size=1, max_size=7), st.data())
def test_dot_tree_behaves_like_the_reference(ref_dt, flat, data):
    keys = sorted(flat)
    flat = {k: v for k, v in flat.items() if not any(o != k and o.startswith(k + ".") for o in keys)}
    mine, ref = DotTree.from_dict(flat), ref_dt.DotTree.from_dict(flat)
    assert dict(mine.to_dict()) == dict(ref.to_dict())
    assert list(mine.to_dict()) == list(ref.to_dict())          # same order
    assert [list(x) for x in mine.unpack()] == [list(x) for x in ref.unpack()]
    assert mine.keys_flat() == ref.keys_flat() and mine.values_flat() == ref.values_flat()
    assert list(mine.keys()) == list(ref.keys()) and mine.len() == ref.len() and mine.len_flat() == ref.len_flat()
    probe = data.draw(st.sampled_from(sorted(flat)))
    assert (probe in mine) == (probe in ref) and mine.get(probe) == ref.get(probe)
    sub = data.draw(st.lists(st.sampled_from(sorted(flat)), unique=True, max_size=3))
    assert dict(mine.filter_keys(sub).to_dict()) == dict(ref.filter_keys(sub).to_dict())
    other = {k: v + 1 for k, v in list(flat.items())[::2]}
    assert mine.to_mapping(DotTree.from_dict(other)) == ref.to_mapping(ref_dt.DotTree.from_dict(other))
    assert dict(mine.map(lambda v: -v).to_dict()) == dict(ref.map(lambda v: -v).to_dict())
    m2, r2 = mine.copy(), ref.copy()
    assert m2.pop(probe) == r2.pop(probe) and dict(m2.to_dict()) == dict(r2.to_dict())
    for tree, cls in ((m2, DotTree), (r2, ref_dt.DotTree)):
        tree.update(cls.from_dict({"zz.new": 1}))
    assert dict(m2.to_dict()) == dict(r2.to_dict())
    for tree in (mine, ref):
        with pytest.raises(ValueError):
            tree.insert(probe, 0)
    # negative numeric indices count back from the largest numeric key
    nums = DotTree.from_dict({"0": "a", "1": "b", "3": "c"}), ref_dt.DotTree.from_dict({"0": "a", "1": "b", "3": "c"})
    assert nums[0].get(-1) == nums[1].get(-1) and nums[0].get(1) == nums[1].get(1) and nums[0].get("3") == nums[1].get("3")
