"""The execution schemes on a CUDA session: the CPU tests of batch serialisation (all IO modes), pipelining, remote
buffers and phased execution are run again with every session placed on the GPU. There the loop bodies are captured into
CUDA graphs and replayed (also loops with carried values: indices and seeds), slab rows and stash slots are indexed on the
device, and ops recorded under `io_tiles()` run on the IO stream. The results must equal what the tests expect of the CPU
backend; counters check that loops were in fact captured and that IO-stream ops ran."""
import numpy as np
import pytest
import torch

import popxl_addons_b200 as addons
from popxl_addons_b200 import xl as popxl
from popxl_addons_b200.xl import ops

pytestmark = pytest.mark.gpu


@pytest.fixture()
def on_cuda(monkeypatch):
    """Sessions asked for the CPU backend run on the GPU; returns counters of captures, replays and IO-stream ops."""
    import popxl_addons_b200.xl.session as sess

    stats = {"captured": 0, "io_ops": 0, "sessions": 0}
    resolve = sess._resolve_device
    monkeypatch.setattr(sess, "_resolve_device", lambda d: resolve("cuda" if (d or "").lower() in ("cpu", "ipu_model") else d))
    capture = sess.Session._capture

    def counting_capture(self, *a, **k):
        state = capture(self, *a, **k)
        stats["captured"] += 1
        return state

    monkeypatch.setattr(sess.Session, "_capture", counting_capture)
    init = sess.Session.__init__

    def counting_init(self, *a, **k):
        init(self, *a, **k)
        stats["sessions"] += 1
        assert self.device.type == "cuda"
        stream = self._io_stream
        if stream is not None:
            wait = stream.wait_stream

            def counted_wait(other, _wait=wait):
                stats["io_ops"] += 1
                return _wait(other)

            stream.wait_stream = counted_wait

    monkeypatch.setattr(sess.Session, "__init__", counting_init)
    return stats


@pytest.mark.parametrize("io_mode", ["compute", "io", "io_overlapped"])
def test_batch_serialisation_on_the_gpu(on_cuda, io_mode):
    import test_transforms as tt

    tt.test_batch_serialisation_forward(io_mode)
    tt.test_batch_serialisation_rows_and_offsets(io_mode)
    tt.test_batch_serialisation_callable_offset(io_mode)
    tt.test_batch_serialised_gradient_equals_plain(io_mode)
    assert on_cuda["sessions"] >= 4
    assert on_cuda["captured"] >= 3, on_cuda  # the micro-batch loops (index and seed are carried values) were captured
    if io_mode != "compute":
        assert on_cuda["io_ops"] > 0, on_cuda  # loads / stores were issued on the IO stream


def test_batch_serialisation_with_sharded_activations_on_the_gpu(on_cuda):
    import test_transforms as tt

    tt.test_batch_serialisation_tp4_dp2_sharded_activations("io_overlapped")
    assert on_cuda["sessions"] >= 1


def test_pipelined_execution_on_the_gpu(on_cuda):
    import test_transforms as tt

    tt.test_pipeline_two_stage_inference()
    tt.test_pipeline_training_with_stash_equals_sequential()
    assert on_cuda["captured"] >= 1, on_cuda  # the steady-state cycle loop (stage hand-offs are carried values)


def test_remote_buffers_and_phased_execution_on_the_gpu(on_cuda):
    import test_session_and_phased as ts

    ts.test_remote_buffers_load_store_graphs()
    ts.test_phased_execution_with_rts()
    ts.test_tensor_parallel_with_rts_subgroup()
    assert on_cuda["sessions"] >= 3


def test_loop_with_carried_values_is_captured_and_continues_across_runs(on_cuda):
    """A counter and an accumulator carried through `repeat`: captured after the first iteration, and a second `run`
    (which replays from the first iteration on) starts again from the values passed in."""
    ir = popxl.Ir()
    with ir.main_graph:
        w = popxl.variable(np.full((4,), 2.0, np.float32), name="w")

        def body(i, acc, w):
            return i + 1, acc + w * ops.cast(i, popxl.float32)

        g = ir.create_graph(body, popxl.constant(0, popxl.int32), popxl.constant(np.zeros(4, np.float32)), w)
        i_out, acc_out = ops.repeat(g, 6, popxl.constant(0, popxl.int32), popxl.constant(np.zeros(4, np.float32)), w)
        si, sa = addons.host_store(i_out), addons.host_store(acc_out)
    with popxl.Session(ir, "cpu") as s:
        for _ in range(2):
            out = s.run()
            assert int(out[si]) == 6
            np.testing.assert_allclose(out[sa], np.full(4, 2.0 * sum(range(6)), np.float32))
    assert on_cuda["captured"] == 1, on_cuda


def test_io_stream_ops_overlap_is_reported(on_cuda):
    """Per-op profile of a program whose loads run under `io_tiles()`: the IO ops are listed as such."""
    ir = popxl.Ir()
    with ir.main_graph:
        buf = popxl.remote_buffer((256, 256), popxl.float32, 4)
        w = popxl.variable(np.eye(256, dtype=np.float32), name="w")
        acc = popxl.variable(np.zeros((256, 256), np.float32), name="acc")
        for i in range(4):
            ops.remote_store(buf, i, w * float(i + 1))
        for i in range(4):
            with popxl.io_tiles():
                x = ops.remote_load(buf, i)
            ops.var_updates.accumulate_(acc, x @ w)
    with popxl.Session(ir, "cpu") as s:
        s.start_profile()
        s.run()
        prof = s.profile_summary()
        assert any(name.endswith("[io]") for name in prof), list(prof)
        np.testing.assert_allclose(s.get_tensor_data(acc), np.eye(256) * 10.0, rtol=1e-6)
    assert on_cuda["io_ops"] >= 4
