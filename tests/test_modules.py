"""Module system: naming, nesting, outlining, graph counts, custom gradients and their error contracts
(behaviours of tests/unit/test_modules.py and test_modules_build_graph.py of popxl_addons)."""
from functools import partial

import numpy as np
import pytest

import popxl_addons_b200 as addons
from popxl_addons_b200 import Module, GraphWithNamedArgs
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops


class Scale(Module):
    def build(self, x):
        scale = self.add_variable_input("scale", partial(np.ones, x.shape), x.dtype)
        return x * scale


class Nested(Module):
    def __init__(self):
        super().__init__()
        self.a = Scale()
        self.b = Scale()

    def build(self, x):
        return self.b(self.a(x))


def test_create_graph_adds_one_graph_and_modules_keep_no_state():
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.ones((2, 2)), popxl.float32)
        m = Scale()
        assert len(ir._pb_ir.getAllGraphs()) == 1
        args, graph = m.create_graph(x)
        assert len(ir._pb_ir.getAllGraphs()) == 2
        assert list(args.to_dict()) == ["scale"] and list(graph.args.to_dict()) == ["scale"]
        assert m._variable_factories.len_flat() == 0
        args2, graph2 = m.create_graph(x)
        assert len(ir.graphs) == 3 and graph2.graph is not graph.graph
        v = args.init()
        (y,) = graph.bind(v).call(x)
        (z,) = graph.bind(args.init()).call(y)
        st = addons.host_store(z)
    np.testing.assert_array_equal(popxl.Session(ir, "cpu").run()[st], np.ones((2, 2)))


def test_nested_modules_are_inlined_with_dotted_names():
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.ones((2, 2)), popxl.float32)
        args, graph = Nested().create_graph(x)
        assert len(ir.graphs) == 2  # inlining adds no graph
        assert sorted(args.to_dict()) == ["a.scale", "b.scale"]
        names = [t.name for t in graph.args.tensors]
        assert any("a/" in n or "a." in n for n in names)
        variables = args.init()
        assert variables.a.scale.name == "a.scale"


def test_outlined_submodule_via_add_variable_inputs():
    class Outlined(Module):
        def build(self, x):
            args, graph = Scale().create_graph(x)
            l1 = graph.bind(self.add_variable_inputs("first", args))
            l2 = graph.bind(self.add_variable_inputs("second", args))
            (x,) = l1.call(x)
            (x,) = l2.call(x)
            return x

    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.full((2,), 3.0), popxl.float32)
        args, graph = Outlined().create_graph(x)
        assert len(ir.graphs) == 3
        assert sorted(args.to_dict()) == ["first.scale", "second.scale"]
        v = args.init()
        (y,) = graph.bind(v).call(x)
        st = addons.host_store(y)
    s = popxl.Session(ir, "cpu")
    s.write_variables_data({v.first.scale: np.full((2,), 2.0, np.float32), v.second.scale: np.full((2,), 5.0, np.float32)})
    np.testing.assert_array_equal(s.run()[st], np.full((2,), 30.0))


def test_from_list_and_from_variable_factories():
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.ones((2,)), popxl.float32)

        class Stack(Module):
            def __init__(self):
                super().__init__()
                self.layers = Module.from_list([Scale(), Scale(), Scale()])

            def build(self, x):
                for layer in self.layers:
                    x = layer(x)
                return self.layers[0](x) if False else x

        args, graph = Stack().create_graph(x)
        assert sorted(args.to_dict()) == ["layers.0.scale", "layers.1.scale", "layers.2.scale"]
        with pytest.raises(AttributeError, match="from_list"):
            iter(Scale())


LINEAR_IN = np.random.RandomState(42).rand(4, 3)
LINEAR_DY = np.random.RandomState(43).rand(4, 3)


class Linear(Module):
    def __init__(self, features):
        super().__init__()
        self.features = features

    def build(self, x):
        self.w = self.add_variable_input("w", partial(np.ones, (x.shape[-1], self.features)), popxl.float32)
        self.b = self.add_variable_input("b", partial(np.zeros, (self.features,)), popxl.float32)
        return (x @ self.w) + self.b


class LinearBuildGrad(Module):
    def __init__(self, features, grad_inlining_error="error", cache=False):
        super().__init__(grad_inlining_error=grad_inlining_error, cache=cache)
        self.features = features

    def build(self, x):
        self.w = self.add_variable_input("w", partial(np.ones, (x.shape[-1], self.features)), popxl.float32)
        self.b = self.add_variable_input("b", partial(np.zeros, (self.features,)), popxl.float32)
        self.aux["x"] = x
        self.aux["w"] = self.w
        return (x @ self.w) + self.b

    def build_grad(self, dLdy):
        dLdx = dLdy @ self.aux["w"].T
        dLdw = (dLdy.T @ self.aux["x"]).T
        self.var_grad["b"] = ops.sum(dLdy, 0)
        self.var_grad["w"] = dLdw
        return dLdx


def _run_linear(module_factory, method):
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(LINEAR_IN, popxl.float32)
        dy = popxl.variable(LINEAR_DY, popxl.float32)
        facts, fwd = module_factory().create_graph(x)
        grad = fwd.autodiff(method=method) if method else addons.autodiff(fwd)
        variables = facts.init()
        info = fwd.bind(variables).call_with_info(x)
        y, *_ = info.outputs
        outs = grad.call(dy, args=grad.grad_graph_info.inputs_dict(info))
        assert len(outs) == len(grad.graph.outputs) == 3
        streams = [addons.host_store(t) for t in (y, *outs)]
    res = popxl.Session(ir, "cpu").run()
    return [res[s] for s in streams], grad, fwd, ir


def test_build_grad_matches_autodiff():
    ref, ref_grad, _, _ = _run_linear(lambda: Linear(3), None)
    got, grad, fwd, ir = _run_linear(lambda: LinearBuildGrad(3), "build_grad")
    forced, _, _, _ = _run_linear(lambda: LinearBuildGrad(3), "autodiff")
    for a, b, c in zip(ref, got, forced):
        np.testing.assert_allclose(a, b, rtol=1e-6)
        np.testing.assert_allclose(a, c, rtol=1e-6)
    info = grad.grad_graph_info
    assert len(grad.graph.inputs) == len(info.expected_inputs) == len(fwd.graph.outputs)
    for g, e in zip(grad.graph.inputs, info.expected_inputs):
        assert g.spec == e.fwd_tensor.spec
    for g, e in zip(grad.graph.outputs, info.expected_outputs):
        assert g.spec == e.fwd_tensor.spec
    kinds = sorted(ec.connection_type.name for ec in info.expected_inputs)
    assert kinds == sorted(ec.connection_type.name for ec in ref_grad.grad_graph_info.expected_inputs)


def test_outlined_build_grad_needs_called_graphs_grad_info():
    class LinearOutlined(Module):
        def build(self, x):
            x = 1 * x
            (y,) = self.call_module(LinearBuildGrad(x.shape[-1]))(x)
            return y

    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(LINEAR_IN, popxl.float32)
        dy = popxl.variable(LINEAR_DY, popxl.float32)
        facts, fwd = LinearOutlined().create_graph(x)
        saved = fwd.called_graphs_grad_info
        assert len(saved) > 0
        fwd.called_graphs_grad_info = {}
        with pytest.raises(Exception, match="marked as unsafe to autodiff"):
            fwd.autodiff()
        fwd.called_graphs_grad_info = saved
        fwd._autodiff_applied = False
        grad = fwd.autodiff()
        v = facts.init()
        info = fwd.bind(v).call_with_info(x)
        y, *_ = info.outputs
        outs = grad.call(dy, args=grad.grad_graph_info.inputs_dict(info))
        streams = [addons.host_store(t) for t in (y, *outs)]
    res = popxl.Session(ir, "cpu").run()
    ref, *_ = _run_linear(lambda: Linear(3), None)
    for a, s in zip(ref, streams):
        np.testing.assert_allclose(a, res[s], rtol=1e-6)


def test_error_contracts():
    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(LINEAR_IN, popxl.float32)
        facts, fwd = LinearBuildGrad(3).create_graph(x)
        manual = GraphWithNamedArgs(fwd.graph, args=fwd.args)
        with pytest.raises(Exception, match="`from_module` is specified"):
            manual.autodiff(method="build_grad")

        class Inlined(Module):
            def __init__(self, mode):
                super().__init__()
                self.linear = LinearBuildGrad(3, grad_inlining_error=mode)

            def build(self, x):
                return self.linear(2 * x)

        with pytest.raises(ValueError, match="grad_inlining_error should be one of"):
            Inlined("")
        with pytest.raises(Exception, match="`build_grad` has been implemented"):
            Inlined("error").create_graph(x)
        with pytest.warns(UserWarning, match="`build_grad` has been implemented"):
            Inlined("warning").create_graph(x)
        Inlined("none").create_graph(x)
        with pytest.raises(ValueError, match="You cannot use graph caching if you have implemented `build_grad`"):
            LinearBuildGrad(3, cache=True)
        grad = fwd.autodiff()
        with pytest.raises(Exception, match="Autodiff has already been applied"):
            fwd.autodiff()
        with pytest.raises(Exception, match="get items within the `build_graph`"):
            LinearBuildGrad(3).aux["x"]

        class MissingVarGrad(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = ops.sum(dLdy, 0)
                return dLdy @ self.aux["w"].T

        with pytest.raises(Exception, match="Not all variable gradients have been specified"):
            MissingVarGrad(3).create_graph(x)[1].autodiff()

        class NotATensor(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = 1.0

        with pytest.raises(TypeError, match="Not a tensor"):
            NotATensor(3).create_graph(x)[1].autodiff()

        class NotAVariable(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["zzz"] = dLdy

        with pytest.raises(KeyError, match="Not a variable"):
            NotAVariable(3).create_graph(x)[1].autodiff()

        class WrongShape(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = dLdy

        with pytest.raises(ValueError, match="Shape or meta-shape of Tensor does not match variable."):
            WrongShape(3).create_graph(x)[1].autodiff()

        class WrongOutShape(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = ops.sum(dLdy, 0)
                self.var_grad["w"] = (dLdy.T @ self.aux["x"]).T
                return ops.sum(dLdy, 0)

        with pytest.raises(ValueError, match="Shape or meta-shape of output Tensor at position 0"):
            WrongOutShape(3).create_graph(x)[1].autodiff()

        class TooMany(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = ops.sum(dLdy, 0)
                self.var_grad["w"] = (dLdy.T @ self.aux["x"]).T
                d = dLdy @ self.aux["w"].T
                return d, d

        with pytest.raises(Exception, match="Too many outputs in the grad graph"):
            TooMany(3).create_graph(x)[1].autodiff()

        class TooFew(LinearBuildGrad):
            def build_grad(self, dLdy):
                self.var_grad["b"] = ops.sum(dLdy, 0)
                self.var_grad["w"] = (dLdy.T @ self.aux["x"]).T

        with pytest.raises(Exception, match="Not all forward graph inputs have been specified"):
            TooFew(3).create_graph(x)[1].autodiff()

        class BadSignature(LinearBuildGrad):
            def build_grad(self, *grads):
                return grads[0]

        with pytest.raises(TypeError, match="method signature must only have a fixed number of positional "
                                            "parameters as inputs."):
            BadSignature(3).create_graph(x)[1].autodiff()
        f2, g2 = LinearBuildGrad(3).create_graph(x)
        with pytest.raises(ValueError, match="is not a output of `fwd_graph`"):
            g2.autodiff(grads_provided=[g2.graph.inputs[0]])
        with pytest.raises(ValueError, match="is not a input of `fwd_graph`"):
            g2.autodiff(grads_required=[g2.graph.outputs[0]])
        with pytest.raises(ValueError, match="do not match the signature"):
            g2.autodiff(grads_provided=[])


def test_route_tensor_into_nested_graphs():
    from popxl_addons_b200.route_tensor import is_subgraph, route_tensor_into_graph

    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.full((2,), 2.0), popxl.float32)
        extra = popxl.variable(np.full((2,), 10.0), popxl.float32)
        inner = ir.create_empty_graph("inner")
        with inner:
            a = popxl.graph_input((2,), popxl.float32, "a")
            popxl.graph_output(a * 1.0)
        outer = ir.create_graph(lambda t: ops.call(inner, t)[0] + 1.0, x)
        (y,) = ops.call(outer, x)
        assert is_subgraph(ir.main_graph, inner) and is_subgraph(outer, inner) and not is_subgraph(inner, outer)
        with inner:
            routed = route_tensor_into_graph(extra)
            inner._outputs[0] = inner._outputs[0] + routed
        other = ir.create_empty_graph("unrelated")
        with pytest.raises(ValueError, match="is not in a known parent graph"):
            route_tensor_into_graph(extra, other)
        with pytest.raises(TypeError):
            route_tensor_into_graph(1.0, inner)
        st = addons.host_store(y)
    np.testing.assert_array_equal(popxl.Session(ir, "cpu").run()[st], np.full((2,), 13.0))


def test_graph_common_normalises_graph_like_keys():
    from popxl_addons_b200.graph_common import normalise_called_graphs_grad_info

    class Scale(addons.Module):
        def build(self, x):
            return x * self.add_variable_input("scale", lambda: np.ones(x.shape, np.float32), x.dtype)

    ir = popxl.Ir()
    with ir.main_graph:
        x = popxl.variable(np.ones((2, 2), np.float32))
        facts, graph = Scale().create_graph(x)
        dgraph = addons.autodiff(graph)
        bound = graph.bind(facts.init())
    info = dgraph.grad_graph_info
    for key, val in ((graph, dgraph), (graph.graph, info), (bound, dgraph)):
        out = normalise_called_graphs_grad_info({key: val})
        assert list(out.keys()) == [graph.graph] and out[graph.graph] is info
    assert normalise_called_graphs_grad_info(None) == {}
