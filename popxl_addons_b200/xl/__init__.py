"""`xl`: the graph-building and execution substrate (the role `popxl` plays for the reference add-ons).

Typical use: `from popxl_addons_b200 import xl as popxl; from popxl_addons_b200.xl import ops`.
"""
from . import dtypes
from .dtypes import (dtype, float64, float32, float16, bfloat16, float8_143, float8_152, int64, int32, int16, int8,
                     uint64, uint32, uint16, uint8, bool_)
from .core import (Ir, Graph, Op, Options, Tensor, Variable, Constant, TensorSpec, TensorByRef, ReplicaGrouping, gcg, gir, gmg,
                   get_current_graph, name_scope, in_sequence, ipu, device, io_tiles, main_tiles, graph_input,
                   graph_output, variable, constant, replica_sharded_variable, LazyInit)
from .buffers import (HostToDeviceStream, DeviceToHostStream, RemoteBuffer, h2d_stream, d2h_stream, remote_buffer,
                      replica_sharded_buffer, remote_variable, remote_replica_sharded_variable)
from . import ops
from . import transforms
from .autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo
from .session import Session
from .ops.control import CallSiteInfo

bool = bool_  # noqa: A001  (popxl exposes the boolean dtype under this name)
Module = object


def create_seeds(seed: int, offset: int = 0, batches_per_step: int = 1, replicas: int = 1):
    """Seed pairs for `replicas` replicas (and `batches_per_step` host transfers): uint32 `(..., 2)`, distinct per
    replica, a pure function of `(seed, offset)`. Counterpart of popxl.create_seeds as used by
    popxl_addons/seed_variable.py:22."""
    import numpy as _np

    rng = _np.random.Generator(_np.random.PCG64([int(seed), int(offset)]))
    shape = ((batches_per_step,) if batches_per_step > 1 else ()) + ((replicas,) if replicas > 1 else ()) + (2,)
    return rng.integers(0, 2 ** 32, size=shape, dtype=_np.uint64).astype(_np.uint32)


# ---- further names and module paths of popxl ------------------------------------------------------------------------
import enum as _enum  # noqa: E402

from . import context, errors, fp8_utils, graph, streams, tensor, utils  # noqa: E402,F401
from .context import get_current_context, get_main_graph, op_debug_context  # noqa: E402,F401
from .transforms import io_tile_exchange, merge_exchange  # noqa: E402,F401

half, double = float16, float64


class TileSet(_enum.Enum):
    """Where an op runs: on the compute stream or on the IO / copy stream (`io_tiles()`)."""

    Compute = "compute"
    IO = "io"
