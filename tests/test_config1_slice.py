"""Minimum end-to-end slice: Linear(64->256)+GELU+Linear(256->64) as a Module, fp32, batch 8, MSE, autodiff, Adam x10,
checkpoint round trip; every number is compared against plain torch."""
import numpy as np
import torch

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops
from popxl_addons_b200.layers import Linear
from popxl_addons_b200.optimizers.adam import AdamOptimizerStep


class MLP(addons.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = Linear(256)
        self.fc2 = Linear(64)

    def build(self, x):
        return self.fc2(ops.gelu(self.fc1(x)))


def build_program(fused_adam=True):
    rng = np.random.RandomState(0)
    x_np = rng.randn(8, 64).astype(np.float32)
    t_np = rng.randn(8, 64).astype(np.float32)
    w1 = (rng.randn(64, 256) * 0.02).astype(np.float32)
    w2 = (rng.randn(256, 64) * 0.02).astype(np.float32)
    ir = popxl.Ir()
    with ir.main_graph:
        streams = addons.InputStreams(x=((8, 64), popxl.float32), t=((8, 64), popxl.float32))
        out_streams = addons.OutputStreams(loss=((), popxl.float32))
        x = ops.host_load(streams.x)
        t = ops.host_load(streams.t)
        facts, graph = MLP().create_graph(x)
        grad = addons.autodiff(graph)
        variables = facts.init()
        info = graph.bind(variables).call_with_info(x)
        y = info.outputs[0]
        diff = y - t
        loss = ops.mean(diff * diff)
        dy = diff * (2.0 / diff.nelms)
        grads = grad.call(dy, args=grad.grad_graph_info.inputs_dict(info))
        by_fwd = dict(zip(grad.grad_graph_info.outputs, grads))
        opt_state = {}
        for name, var in variables.to_dict().items():
            g = by_fwd[graph.args.to_dict()[name]]
            ofacts, ograph = AdamOptimizerStep(fused=fused_adam).create_graph(
                var, g, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-5, weight_decay=0.0, first_order_dtype=popxl.float32)
            ostate = ofacts.init(prefix=f"adam.{name}")
            ograph.bind(ostate).call(var, g)
            opt_state[name] = ostate
        ops.host_store(out_streams.loss, loss)
    state = addons.NamedTensors(model=variables)
    for name, s in opt_state.items():
        state.insert(f"adam.{name.replace('.', '_')}", s, overwrite=True)
    return ir, streams, out_streams, state, variables, (x_np, t_np, w1, w2)


def torch_reference(x_np, t_np, w1, w2, steps):
    tw1 = torch.tensor(w1, requires_grad=True)
    tw2 = torch.tensor(w2, requires_grad=True)
    tb1 = torch.zeros(256, requires_grad=True)
    tb2 = torch.zeros(64, requires_grad=True)
    opt = torch.optim.AdamW([tw1, tb1, tw2, tb2], lr=1e-3, betas=(0.9, 0.999), eps=1e-5, weight_decay=0.0)
    x, t = torch.tensor(x_np), torch.tensor(t_np)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        y = torch.nn.functional.gelu(x @ tw1 + tb1) @ tw2 + tb2
        loss = ((y - t) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, tw1.detach().numpy(), tw2.detach().numpy()


def run(fused, tmp_path=None):
    ir, streams, out_streams, state, variables, (x_np, t_np, w1, w2) = build_program(fused)
    session = addons.TaskSession(streams, out_streams, state, 2, ir, "cpu")
    session.write_variables_data({variables.fc1.weight: w1, variables.fc2.weight: w2})
    losses = []
    with session:
        for _ in range(10):
            out = session.run({streams.x: x_np, streams.t: t_np})
            losses.append(float(out[out_streams.loss]))
    return session, losses, variables, (x_np, t_np, w1, w2)


def test_training_matches_torch_adamw():
    for fused in (True, False):
        session, losses, variables, data = run(fused)
        ref_losses, rw1, rw2 = torch_reference(*data, steps=10)
        np.testing.assert_allclose(losses, ref_losses, rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(session.get_tensor_data(variables.fc1.weight), rw1, atol=2e-5)
        np.testing.assert_allclose(session.get_tensor_data(variables.fc2.weight), rw2, atol=2e-5)
        assert losses[-1] < losses[0]


def test_checkpoint_round_trip(tmp_path):
    session, losses, variables, data = run(True)
    ckpt = str(tmp_path / "ckpt")
    session.save_checkpoint(ckpt)
    import os

    assert os.path.exists(os.path.join(ckpt, "model", "model.fc1.weight.npz"))
    assert os.path.exists(os.path.join(ckpt, "session_info.json"))
    with np.load(os.path.join(ckpt, "model", "model.fc1.weight.npz")) as z:
        assert "model.fc1.weight" in z.files
    before = session.get_named_tensors_data().to_dict()
    # a fresh session restored from the checkpoint continues identically
    ir, streams, out_streams, state, variables2, _ = build_program(True)
    s2 = addons.TaskSession(streams, out_streams, state, 2, ir, "cpu")
    s2.load_checkpoint(ckpt)
    assert s2.session_state["steps"] == 10
    after = s2.get_named_tensors_data().to_dict()
    assert set(before) == set(after)
    for k in before:
        np.testing.assert_array_equal(before[k], after[k])
    x_np, t_np = data[0], data[1]
    a = session.run({session.inputs.x: x_np, session.inputs.t: t_np})[session.outputs.loss]
    b = s2.run({streams.x: x_np, streams.t: t_np})[out_streams.loss]
    np.testing.assert_allclose(a, b, rtol=1e-6)
