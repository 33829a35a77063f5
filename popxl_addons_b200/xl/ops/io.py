"""Host streams, remote-buffer access and device-to-device copies.

* `host_load` / `host_store` move one micro-batch between pinned host memory and the device on the IO stream.
* `remote_load` / `remote_store` read / write one row of a `RemoteBuffer` slab (device HBM by default, pinned host
  memory for offload) at a run-time index.
* `ipu_copy` moves a tensor to another device slot (pipeline stage boundary): NCCL send/recv between ranks.

Parity: popxl `ops.host_load/host_store/remote_load/remote_store`, `Tensor.copy_to_ipu` as used by
popxl_addons/ops/streams.py:13-23, remote.py:119-222, transforms/pipelining.py:184-191.
"""
from typing import Optional, Union

from ..core import Tensor, constant, current_device
from .. import dtypes as _dt
from ..opdef import OpDef, emit, emit1


def _special_host_load(ex, op, env):
    env[op.outputs[0]] = ex.host_load(op.attrs["stream"])


OpDef("host_load", special=_special_host_load,
      infer=lambda op: [(op.attrs["stream"].shape, op.attrs["stream"].dtype, op.attrs["stream"].meta_shape)])


def host_load(h2d_stream, name: Optional[str] = None) -> Tensor:
    return emit("host_load", [], {"stream": h2d_stream}, [name or h2d_stream.name])[0]


def _special_host_store(ex, op, env):
    ex.host_store(op.attrs["stream"], env[op.inputs[0]])


OpDef("host_store", special=_special_host_store, infer=lambda op: [])


def host_store(d2h_stream, t: Tensor) -> None:
    if tuple(d2h_stream.shape) != tuple(t.shape):
        raise ValueError(f"Tensor shape {t.shape} does not match stream shape {d2h_stream.shape}")
    if d2h_stream.dtype != t.dtype:
        raise ValueError(f"Tensor dtype {t.dtype} does not match stream dtype {d2h_stream.dtype}")
    emit("host_store", [t], {"stream": d2h_stream})


def _offset_tensor(offset) -> Tensor:
    if isinstance(offset, Tensor):
        return offset
    return constant(int(offset), _dt.int32, "offset")


def _special_remote_load(ex, op, env):
    env[op.outputs[0]] = ex.remote_load(op.attrs["buffer"], env[op.inputs[0]])


def _special_remote_store(ex, op, env):
    ex.remote_store(op.attrs["buffer"], env[op.inputs[0]], env[op.inputs[1]])


OpDef("remote_load", special=_special_remote_load,
      infer=lambda op: [(op.attrs["buffer"].tensor_shape, op.attrs["buffer"].tensor_dtype,
                         op.attrs["buffer"].meta_shape)])
OpDef("remote_store", special=_special_remote_store, infer=lambda op: [])


def remote_load(remote_buffer, offset: Union[int, Tensor], name: Optional[str] = None) -> Tensor:
    return emit("remote_load", [_offset_tensor(offset)], {"buffer": remote_buffer}, [name or "remote_load"])[0]


def remote_load_(remote_buffer, offset, t: Tensor) -> Tensor:
    return remote_load(remote_buffer, offset)


def remote_store(remote_buffer, offset: Union[int, Tensor], t: Tensor) -> None:
    if t.nelms != _prod(remote_buffer.tensor_shape):
        raise ValueError(f"Tensor of shape {t.shape} does not fit buffer rows of shape {remote_buffer.tensor_shape}")
    if t.dtype != remote_buffer.tensor_dtype:
        raise ValueError(f"Tensor dtype {t.dtype} does not match buffer dtype {remote_buffer.tensor_dtype}")
    emit("remote_store", [_offset_tensor(offset), t], {"buffer": remote_buffer})


def _prod(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _special_ipu_copy(ex, op, env):
    env[op.outputs[0]] = ex.device_copy(env.get(op.inputs[0]), op)


def _vjp_ipu_copy(ctx, op, gs):
    return [ipu_copy(gs[0], op.attrs["source"], op.attrs["destination"])]


OpDef("ipu_copy", special=_special_ipu_copy, vjp=_vjp_ipu_copy,
      infer=lambda op: [(op.inputs[0].shape, op.inputs[0].dtype, op.inputs[0].meta_shape)])


def ipu_copy(t: Tensor, destination: int, source: Optional[int] = None) -> Tensor:
    src = t.device_index if source is None else int(source)
    outs = emit("ipu_copy", [t], {"source": src, "destination": int(destination)}, [t.id.split("/")[-1] + "_c"])
    outs[0].device_index = int(destination)
    return outs[0]
