"""Graph substrate: Ir / Graph / Op / Tensor / TensorSpec / ReplicaGrouping and the build-time context stack.

A model is described by running ordinary Python (`Module.build`, user functions) against symbolic `Tensor`s; every
operator call appends an `Op` to the graph on top of the context stack. Nothing touches a device while building: shapes
and dtypes are inferred by running each op's reference implementation on torch *meta* tensors. A `Session` later
interprets the recorded graphs on real `torch.Tensor`s (CPU for tests and oracles, CUDA for production, one process
per GPU).

This file supplies the part of the `popxl` surface that popxl_addons relies on (module.py:8-12,
variable_factory.py:9-14, transforms/*.py): `Ir`, `Graph`, `Tensor`, `TensorSpec`, `TensorByRef`, `variable`,
`constant`, `graph_input`, `graph_output`, `name_scope`, `in_sequence`, `ipu`, `io_tiles`, `gcg/gir/gmg`,
`ReplicaGrouping` and op-created hooks (transforms/pipelining.py:464-470).
"""
import contextlib
import inspect
import dataclasses
import itertools
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import dtypes as _dt
from .dtypes import dtype

# ---------------------------------------------------------------------------------------------------------------
# build-time context
# ---------------------------------------------------------------------------------------------------------------


class _BuildState:
    def __init__(self):
        self.graphs: List["Graph"] = []
        self.scopes: List[str] = []
        self.sequence: List[Any] = []
        self.devices: List[int] = []
        self.tile_sets: List[str] = []
        self.merge_exchange: int = 0


_STATE = _BuildState()


def gcg() -> "Graph":
    """Graph currently being built."""
    if not _STATE.graphs:
        raise RuntimeError("Trying to access a graph, but no graph has been selected. Hint - try performing the "
                           "operations in a context of `with graph:`")
    return _STATE.graphs[-1]


def gir() -> "Ir":
    return gcg().ir


def gmg() -> "Graph":
    return gir().main_graph


def get_current_graph() -> "Graph":
    return gcg()


@contextlib.contextmanager
def name_scope(name: str):
    """Prefix names of tensors created inside with `name/`."""
    _STATE.scopes.append(name)
    try:
        yield
    finally:
        _STATE.scopes.pop()


def current_scope() -> str:
    return "/".join(_STATE.scopes)


@contextlib.contextmanager
def in_sequence(enabled: Union[bool, str] = True):
    """Ops are always executed in recorded order by the interpreter, so this only records the annotation."""
    _STATE.sequence.append(enabled)
    try:
        yield
    finally:
        _STATE.sequence.pop()


@contextlib.contextmanager
def ipu(index: Optional[int]):
    """Place ops on device slot `index` (a pipeline stage's GPU). Kept under the reference's name for API parity.
    `ipu(None)` suspends an enclosing placement: ops created inside follow their operands, or the call site when they
    belong to a graph that is called from several slots."""
    _STATE.devices.append(None if index is None else int(index))
    try:
        yield
    finally:
        _STATE.devices.pop()


device = ipu


def current_device() -> int:
    return _STATE.devices[-1] if _STATE.devices and _STATE.devices[-1] is not None else 0


@contextlib.contextmanager
def io_tiles():
    """Ops inside run on the copy/IO stream instead of the compute stream (overlapped IO)."""
    _STATE.tile_sets.append("io")
    try:
        yield
    finally:
        _STATE.tile_sets.pop()


@contextlib.contextmanager
def main_tiles():
    _STATE.tile_sets.append("compute")
    try:
        yield
    finally:
        _STATE.tile_sets.pop()


def current_tile_set() -> str:
    return _STATE.tile_sets[-1] if _STATE.tile_sets else "compute"


# ---------------------------------------------------------------------------------------------------------------
# ReplicaGrouping
# ---------------------------------------------------------------------------------------------------------------


class ReplicaGrouping:
    """Partition of the `num_replicas` replicas (= ranks) into equally sized groups.

    With `(stride s, group_size g)` replica `r` belongs to `{b*s*g + (r mod s) + j*s : j < g}`, `b = r div (s*g)`;
    its position inside the group is `(r mod s*g) div s`. A grouping can also be given as an explicit assignment
    (group index per replica), which is what `transpose()` produces when the complement is not expressible as
    (stride, size). On one NVSwitch box every grouping costs the same, so a group is just a rank list.
    """

    def __init__(self, num_replicas: int, stride: int = 1, group_size: Optional[int] = None,
                 assignment: Optional[Sequence[int]] = None):
        self.num_replicas = int(num_replicas)
        if assignment is not None:
            self._assignment = [int(a) for a in assignment]
            assert len(self._assignment) == self.num_replicas
            self._stride, self._group_size = None, None
            sizes = {}
            for a in self._assignment:
                sizes[a] = sizes.get(a, 0) + 1
            if len(set(sizes.values())) != 1:
                raise ValueError("All replica groups must have the same size")
            self._group_size = next(iter(sizes.values()))
            self._canonicalise()
        else:
            if group_size is None:
                group_size = self.num_replicas // stride
            stride, group_size = int(stride), int(group_size)
            if group_size == 1:
                stride = 1
            if stride < 1 or group_size < 1 or self.num_replicas % (stride * group_size) != 0:
                raise ValueError(
                    f"Invalid replica grouping: stride={stride} group_size={group_size} "
                    f"num_replicas={self.num_replicas}")
            self._stride, self._group_size = stride, group_size
            self._assignment = [self._group_of(r) for r in range(self.num_replicas)]

    def _group_of(self, r: int) -> int:
        s, g = self._stride, self._group_size
        return (r // (s * g)) * s + (r % s)

    def _canonicalise(self):
        """If an explicit assignment equals some (stride, size) grouping, adopt that form (makes equality simple)."""
        n, g = self.num_replicas, self._group_size
        for s in range(1, n + 1):
            if n % (s * g) != 0:
                continue
            if g == 1 and s != 1:
                continue
            cand = [(r // (s * g)) * s + (r % s) for r in range(n)]
            if _same_partition(cand, self._assignment):
                self._stride = s
                self._assignment = cand
                return

    # -- properties -------------------------------------------------------------------------------------------
    @property
    def stride(self) -> int:
        if self._stride is None:
            raise ValueError("This replica grouping is defined by an explicit assignment and has no stride")
        return self._stride

    @property
    def group_size(self) -> int:
        return self._group_size

    @property
    def num_groups(self) -> int:
        return self.num_replicas // self._group_size

    @property
    def assignment(self) -> List[int]:
        return list(self._assignment)

    @property
    def is_const(self) -> bool:
        return self._stride is None

    @property
    def const_rg(self):
        return self

    @property
    def groups(self) -> List[List[int]]:
        """Rank lists, ordered by group index; members in increasing replica order (= shard order)."""
        out: Dict[int, List[int]] = {}
        for r, a in enumerate(self._assignment):
            out.setdefault(a, []).append(r)
        return [out[k] for k in sorted(out)]

    def group_of(self, replica: int) -> List[int]:
        a = self._assignment[replica]
        return [r for r, x in enumerate(self._assignment) if x == a]

    def group_index(self, replica: int) -> int:
        return self._assignment[replica]

    def index_in_group(self, replica: int) -> int:
        return self.group_of(replica).index(replica)

    def transpose(self) -> "ReplicaGrouping":
        """Complementary grouping: replicas at the same position of different groups form the new groups.
        (TP grouping <-> DP grouping.)"""
        assign = [self.index_in_group(r) for r in range(self.num_replicas)]
        return ReplicaGrouping(self.num_replicas, assignment=assign)

    def __eq__(self, other):
        return (isinstance(other, ReplicaGrouping) and self.num_replicas == other.num_replicas
                and _same_partition(self._assignment, other._assignment))

    def __hash__(self):
        return hash((self.num_replicas, tuple(tuple(g) for g in self.groups)))

    def __repr__(self):
        if self._stride is not None:
            return (f"ReplicaGrouping(num_replicas={self.num_replicas}, stride={self._stride}, "
                    f"group_size={self._group_size}, num_groups={self.num_groups})")
        return f"ReplicaGrouping(num_replicas={self.num_replicas}, assignment={self._assignment})"


def _same_partition(a: Sequence[int], b: Sequence[int]) -> bool:
    fwd, bwd = {}, {}
    for x, y in zip(a, b):
        if fwd.setdefault(x, y) != y or bwd.setdefault(y, x) != x:
            return False
    return True


# ---------------------------------------------------------------------------------------------------------------
# Tensors
# ---------------------------------------------------------------------------------------------------------------


class TensorSpec:
    """Shape + dtype (+ full `meta_shape` for a replica-sharded tensor): enough to create a graph input."""

    def __init__(self, shape: Iterable[int], dtype: dtype, meta_shape: Optional[Iterable[int]] = None):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = _dt.dtype.as_dtype(dtype)
        self.meta_shape = tuple(int(s) for s in meta_shape) if meta_shape else ()

    @property
    def nelms(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    def __repr__(self):
        ms = f", meta_shape={self.meta_shape}" if self.meta_shape else ""
        return f"TensorSpec(shape={self.shape}, dtype={self.dtype}{ms})"

    def __eq__(self, other):
        return (isinstance(other, TensorSpec) and self.shape == other.shape and self.dtype == other.dtype
                and self.meta_shape == other.meta_shape)

    def __hash__(self):
        return hash((self.shape, self.dtype, self.meta_shape))


class Tensor:
    """Symbolic value in a graph. Python operators record ops; identity (not value) defines equality/hashing."""

    _counter = itertools.count()
    kind = "act"

    def __init__(self, graph: "Graph", shape, dtype_: dtype, name: Optional[str] = None, meta_shape=None,
                 producer: Optional["Op"] = None):
        self.graph = graph
        self._shape = tuple(int(s) for s in shape)
        self._dtype = _dt.dtype.as_dtype(dtype_)
        self.meta_shape = tuple(int(s) for s in meta_shape) if meta_shape else ()
        self.producer = producer
        self.uid = next(Tensor._counter)
        base = name if name else "t"
        scope = current_scope()
        full = f"{scope}/{base}" if scope else base
        self.id = graph._unique_tensor_id(full)
        # an op's outputs live where the op runs; other tensors where the enclosing `ipu(...)` context says
        self.device_index = producer.device_index if producer is not None else current_device()
        self.tile_set = current_tile_set()
        graph._tensors.append(self)

    # -- basic properties ---------------------------------------------------------------------------------------
    @property
    def name(self) -> str:
        return self.id

    @property
    def shape(self) -> Tuple[int, ...]:
        return self._shape

    @property
    def dtype(self) -> dtype:
        return self._dtype

    @property
    def ir(self) -> "Ir":
        return self.graph.ir

    @property
    def spec(self) -> TensorSpec:
        return TensorSpec(self._shape, self._dtype, self.meta_shape)

    @property
    def nelms(self) -> int:
        return int(np.prod(self._shape)) if self._shape else 1

    @property
    def rank(self) -> int:
        return len(self._shape)

    @property
    def ipu(self) -> int:
        return self.device_index

    @property
    def in_sync_with(self):
        return self

    def strides(self, shape=None) -> Tuple[int, ...]:
        """Strides in bytes of a contiguous array of `shape` (default: this tensor's shape) and this dtype."""
        shape = tuple(self.shape if shape is None else shape)
        out, step = [], _dt.itemsize(self.dtype) if hasattr(_dt, "itemsize") else self.dtype.as_torch().itemsize
        for n in reversed(shape):
            out.append(step)
            step *= int(n)
        return tuple(reversed(out))

    @property
    def location_info(self):
        """`(device slot, tile set)` the tensor was created on."""
        return self.device_index, getattr(self.producer, "tile_set", "compute") if self.producer is not None else "compute"

    @property
    def in_sync_with_ipu(self) -> bool:
        """Host data of a variable is written to the device when the session is created and read back on request: the
        two never drift apart silently."""
        return True

    def __repr__(self):
        ms = f", meta_shape={self.meta_shape}" if self.meta_shape else ""
        return f"Tensor[{self.id} {self._dtype} {self._shape}{ms}]"

    def __hash__(self):
        return self.uid

    def __eq__(self, other):
        return self is other

    def __ne__(self, other):
        return self is not other

    def __len__(self):
        if not self._shape:
            raise TypeError("len() of a 0-d tensor")
        return self._shape[0]

    # -- operators (defer to the op library) --------------------------------------------------------------------
    def _ops(self):
        from . import ops

        return ops

    def _lift(self, other) -> "Tensor":
        if isinstance(other, Tensor):
            return other
        dt = self._dtype
        if isinstance(other, (bool, int, float)):
            return constant(other, dt)
        return constant(other, dt if np.asarray(other).dtype.kind == np.dtype(dt.as_numpy()).kind else None)

    def __add__(self, o):
        return self._ops().add(self, self._lift(o))

    def __radd__(self, o):
        return self._ops().add(self._lift(o), self)

    def __sub__(self, o):
        return self._ops().sub(self, self._lift(o))

    def __rsub__(self, o):
        return self._ops().sub(self._lift(o), self)

    def __mul__(self, o):
        return self._ops().mul(self, self._lift(o))

    def __rmul__(self, o):
        return self._ops().mul(self._lift(o), self)

    def __truediv__(self, o):
        return self._ops().div(self, self._lift(o))

    def __rtruediv__(self, o):
        return self._ops().div(self._lift(o), self)

    def __mod__(self, o):
        return self._ops().fmod(self, self._lift(o))

    def __pow__(self, o):
        return self._ops().pow(self, self._lift(o))

    def __neg__(self):
        return self._ops().negate(self)

    def __matmul__(self, o):
        return self._ops().matmul(self, o)

    def __rmatmul__(self, o):
        return self._ops().matmul(self._lift(o), self)

    def __getitem__(self, key):
        return self._ops().subscript(self, key)

    def __iadd__(self, o):
        return self._ops().add_(self, self._lift(o))

    @property
    def T(self) -> "Tensor":
        return self._ops().transpose(self)

    @property
    def T_(self) -> "Tensor":
        return self._ops().transpose(self)

    def transpose(self, permutation: Optional[Iterable[int]] = None) -> "Tensor":
        return self._ops().transpose(self, permutation)

    transpose_ = transpose

    def reshape(self, shape: Iterable[int]) -> "Tensor":
        return self._ops().reshape(self, shape)

    reshape_ = reshape

    def flatten(self) -> "Tensor":
        return self._ops().reshape(self, (-1,))

    flatten_ = flatten

    def detach(self) -> "Tensor":
        return self._ops().detach(self)

    detach_ = detach

    def copy_to_ipu(self, destination: int, source: Optional[int] = None) -> "Tensor":
        return self._ops().ipu_copy(self, destination, source)

    def diag(self):
        raise NotImplementedError


class Variable(Tensor):
    """Persistent tensor owned by the main graph. Replicas in the same group of `replica_grouping` hold identical
    values; with `num_groups > 1` the host-side array has a leading `num_groups` axis."""

    kind = "variable"

    def __init__(self, graph, shape, dtype_, name=None, meta_shape=None, replica_grouping=None,
                 remote_buffer=None, entry: Optional[int] = None, shard_group=None):
        super().__init__(graph, shape, dtype_, name, meta_shape)
        self.replica_grouping: ReplicaGrouping = replica_grouping or graph.ir.replica_grouping()
        self.remote_buffer = remote_buffer
        self.entry = entry
        # group across which a replica-sharded variable is split (None: not sharded)
        self.shard_group: Optional[ReplicaGrouping] = shard_group
        self.retrieval_mode = "one_per_group"
        # replica group whose members may access this variable's storage directly over NVLink (the session then
        # places it in that group's symmetric-memory arena when it runs one process per GPU)
        self.symmetric_group: Optional[ReplicaGrouping] = None
        # the host array when the variable was initialised from a numpy memmap: host reads of the variable are written
        # through to it and return it
        self._memmap_arr = None

    @property
    def shape_on_host(self) -> Tuple[int, ...]:
        base = self.meta_shape if (self.meta_shape and self.shard_group is not None) else self._shape
        if self.replica_grouping.num_groups > 1:
            return (self.replica_grouping.num_groups, *base)
        return tuple(base)

    @property
    def shape_on_replica(self) -> Tuple[int, ...]:
        return self._shape

    @property
    def is_remote(self) -> bool:
        return self.remote_buffer is not None


class Constant(Tensor):
    kind = "constant"

    def __init__(self, graph, data: torch.Tensor, name=None):
        super().__init__(graph, tuple(data.shape), _dt.dtype.as_dtype(data.dtype), name)
        self.data = data


class TensorByRef(Tensor):
    """Annotation type: a `create_graph` parameter annotated with it becomes a by-reference graph input."""


# ---------------------------------------------------------------------------------------------------------------
# Ops and graphs
# ---------------------------------------------------------------------------------------------------------------


class Op:
    """One recorded operation: `outputs = opdef(inputs, **attrs)`."""

    __slots__ = ("opdef", "inputs", "outputs", "attrs", "graph", "name", "device_index", "device_explicit", "tile_set", "stage",
                 "debug", "uid", "id", "attrs_hint", "__weakref__")
    _counter = itertools.count()

    def __init__(self, opdef, inputs, attrs, graph):
        self.opdef = opdef
        self.inputs: List[Tensor] = list(inputs)
        self.outputs: List[Tensor] = []
        self.attrs: Dict[str, Any] = attrs
        self.graph = graph
        self.name = opdef.name
        # device slot: the enclosing `ipu(...)` context if there is one; otherwise the op follows its operands
        # (ops that transforms create outside any context, e.g. stash updates or gradient accumulation)
        self.device_explicit = bool(_STATE.devices) and _STATE.devices[-1] is not None
        if self.device_explicit:
            self.device_index = _STATE.devices[-1]
        else:
            on = [t.device_index for t in self.inputs if not isinstance(t, Constant)]
            self.device_index = max(on) if on else 0
        self.tile_set = current_tile_set()
        self.stage = None
        self.debug = None
        self.attrs_hint = None
        self.uid = next(Op._counter)
        self.id = graph.ir._next_op_id() if graph is not None else self.uid  # per Ir, from 100, in creation order

    @property
    def op_type(self) -> str:
        return self.opdef.name

    def opid(self):
        return self.opdef.name

    def __repr__(self):
        ins = ", ".join(t.id for t in self.inputs)
        outs = ", ".join(t.id for t in self.outputs)
        return f"{outs} = {self.opdef.name}({ins})"


class Graph:
    def __init__(self, ir: "Ir", name: str):
        self.ir = ir
        self.name = name
        self.id = name
        self._inputs: List[Tensor] = []
        self._outputs: List[Tensor] = []
        self._by_ref: set = set()
        self.ops: List[Op] = []
        self._tensors: List[Tensor] = []
        self._ids: Dict[str, int] = {}
        self._hooks: Dict[int, Callable] = {}
        self._hook_ids = itertools.count()
        self.can_autodiff = True
        self.hints: Dict[str, Any] = {}

    # -- context ------------------------------------------------------------------------------------------------
    def __enter__(self):
        _STATE.graphs.append(self)
        return self

    def __exit__(self, *exc):
        _STATE.graphs.pop()
        return False

    def _unique_tensor_id(self, name: str) -> str:
        n = self._ids.get(name, 0)
        self._ids[name] = n + 1
        return name if n == 0 else f"{name}__{n}"

    # -- structure ----------------------------------------------------------------------------------------------
    @property
    def inputs(self) -> Tuple[Tensor, ...]:
        return tuple(self._inputs)

    @property
    def outputs(self) -> Tuple[Tensor, ...]:
        return tuple(self._outputs)

    @property
    def tensors(self) -> Tuple[Tensor, ...]:
        return tuple(self._tensors)

    @property
    def variables(self) -> Tuple[Variable, ...]:
        return tuple(t for t in self._tensors if isinstance(t, Variable))

    @property
    def _pb_graph(self) -> "_PbGraph":
        return _PbGraph(self)

    @property
    def _by_ref_inputs(self) -> set:
        """The graph inputs that were declared by reference (popxl keeps them under this name)."""
        return self._by_ref

    @property
    def constants(self) -> Tuple[Constant, ...]:
        return tuple(t for t in self._tensors if isinstance(t, Constant))

    @property
    def inputs_by_name(self) -> Dict[str, Tensor]:
        return {t.name: t for t in self._inputs}

    @property
    def main_graph(self) -> "Graph":
        return self.ir.main_graph

    def is_by_ref(self, t: Tensor) -> bool:
        return t in self._by_ref

    def get_main_graph(self) -> "Graph":
        return self.ir.main_graph

    def get_tensor(self, tensor_id: str) -> Tensor:
        """The tensor of this graph with the given id."""
        for t in self._tensors:
            if t.id == tensor_id:
                return t
        raise KeyError(f"There is no tensor with id '{tensor_id}' in the graph {self.name}")

    def get_variable(self, tensor_id: str) -> Variable:
        t = self.get_tensor(tensor_id)
        if not isinstance(t, Variable):
            raise TypeError(f"Tensor '{tensor_id}' is not a variable")
        return t

    def _create_tensor_id(self, name: Optional[str] = None) -> str:
        """A tensor id of this graph that is not in use yet, derived from `name`."""
        return self._unique_tensor_id(name or "t")

    def get_input_tensors(self):
        return self.inputs

    def get_output_tensors(self):
        return self.outputs

    def called_graphs(self) -> List["Graph"]:
        seen, out = set(), []
        for op in self.ops:
            for key in ("graph", "body"):
                g = op.attrs.get(key)
                if isinstance(g, Graph) and id(g) not in seen:
                    seen.add(id(g))
                    out.append(g)
        return out

    def __contains__(self, t) -> bool:
        return isinstance(t, Tensor) and t.graph is self

    # -- op hooks (used by the pipelining transform to see every op as it is created) ---------------------------
    def register_op_created_hook(self, fn: Callable[[Op], None]) -> int:
        h = next(self._hook_ids)
        self._hooks[h] = fn
        return h

    def remove_op_created_hook(self, handle: int):
        self._hooks.pop(handle, None)

    def _op_created(self, op: Op):
        for fn in list(self._hooks.values()):
            fn(op)

    def __repr__(self):
        return f"Graph[{self.name}]"

    def __hash__(self):
        return id(self)

    def __eq__(self, other):
        return self is other

    def print_ops(self) -> str:
        return "\n".join(repr(o) for o in self.ops)


@dataclasses.dataclass
class Options:
    """Typed run-time options of an `Ir` (read by the `Session` that executes it). Every field can be overridden from the
    environment (`XL_<FIELD NAME IN CAPITALS>`, e.g. `XL_NATIVE_KERNELS=0`); the reference has no configuration system
    beyond constructor arguments and a few environment variables (popxl_addons/debugging.py:21,
    named_replica_grouping.py:78-85)."""

    native_kernels: bool = True        # run the sm_100a kernels on CUDA sessions (False: torch reference everywhere)
    cuda_graphs: bool = True           # capture `repeat(..., cuda_graph=True)` bodies and replay them
    capture_loops: bool = True         # also capture every other `repeat` body (>= 3 iterations) that holds no op which
                                       # reads a device value on the host; a body whose capture fails runs eagerly
    profile_ops: bool = False          # time every op (CUDA events / perf_counter) into `Session.profile`
    nvtx: bool = False                 # NVTX range per op, named `<graph>/<op>`
    collective_timeout_s: float = 600.0  # process-group timeout: a collective that waits longer ends with an error
    hints: Dict[str, Any] = dataclasses.field(default_factory=dict)  # recorded planner hints (memory proportion, fc pass)

    @classmethod
    def from_env(cls) -> "Options":
        import os

        o = cls()
        for f in dataclasses.fields(cls):
            raw = os.environ.get("XL_" + f.name.upper())
            if raw is None or f.name == "hints":
                continue
            setattr(o, f.name, raw.lower() not in ("0", "false", "no", "") if f.type is bool or f.type == "bool"
                    else float(raw))
        # older spellings
        if os.environ.get("XL_NATIVE") is not None:
            o.native_kernels = os.environ["XL_NATIVE"] != "0"
        return o

    # dict-style access: typed fields by name, anything else is kept as a hint (what the IPU planner knobs of the
    # reference become here: recorded, readable, without effect on the result)
    def __getitem__(self, key):
        return getattr(self, key) if key in self._fields() else self.hints[key]

    def __setitem__(self, key, value):
        if key in self._fields():
            setattr(self, key, value)
        else:
            self.hints[key] = value

    def __contains__(self, key):
        return key in self._fields() or key in self.hints

    def get(self, key, default=None):
        return self[key] if key in self else default

    def setdefault(self, key, default=None):
        if key not in self:
            self[key] = default
        return self[key]

    def _fields(self):
        return {f.name for f in dataclasses.fields(self)} - {"hints"}


_PB_TYPE_NAMES = {"matmul": "MatMul", "add": "Add", "sub": "Sub", "mul": "Mul", "div": "Div",
                  "group_norm": "GroupNormalization", "call": "Call", "repeat": "Loop", "host_load": "HostLoad",
                  "host_store": "HostStore", "ipu_copy": "IpuCopy", "remote_load": "RemoteLoad",
                  "remote_store": "RemoteStore", "accumulate_": "Accumulate", "accumulate_mean_": "Accumulate",
                  "accumulate_moving_average_": "Accumulate", "accumulate_moving_average_square_": "Accumulate",
                  "all_reduce": "ReplicatedAllReduce", "reduce_scatter": "ReplicatedReduceScatter",
                  "all_gather": "ReplicatedAllGather", "init": "Init"}


def pb_op_type(op: "Op") -> str:
    """Op type under popart's naming (`MatMul`, `Add`, `Call`, ...): CamelCase of the op name where popart has none."""
    name = op.opdef.name
    if name in _PB_TYPE_NAMES:
        return _PB_TYPE_NAMES[name]
    return "".join(p.capitalize() for p in name.rstrip("_").split("_")) + ("Inplace" if name.endswith("_") else "")


class _PbTensorInfo:
    def __init__(self, t):
        self._t = t

    def shape(self):
        return list(self._t.shape)

    def nelms(self):
        return self._t.nelms


class _PbTensor:
    def __init__(self, t):
        self._t = t
        self.id = t.id
        self.info = _PbTensorInfo(t)


class _PbOp:
    """Read-only view of an op with the accessors of popart's `Op` that scripts written for the reference use."""

    def __init__(self, op: "Op"):
        self._op = op
        self.id = op.id

    def opType(self) -> str:
        return pb_op_type(self._op)

    def name(self) -> str:
        return self._op.name

    def getInputTensors(self):
        return [_PbTensor(t) for t in self._op.inputs]

    def getOutputTensors(self):
        return [_PbTensor(t) for t in self._op.outputs]

    def debugName(self) -> str:
        return f"{self.opType()}.{self.id}"


class _PbCallOp(_PbOp):
    def getCalledGraph(self):
        return _PbGraph(self._op.attrs["graph"])


class _PbLoopOp(_PbCallOp):
    def getTripCountValue(self) -> int:
        return int(self._op.attrs.get("count", 1))


class _PbMatMulOp(_PbOp):
    """Matmul-class ops carry the 'keep a pre-transposed weight for the backward passes' flag."""

    def useFullyConnectedPass(self) -> bool:
        per_op = self._op.graph.hints.get("fc_pass", {})
        if self._op.uid in per_op:
            return bool(per_op[self._op.uid])
        return bool(self._op.graph.ir.options.hints.get("use_fc_pass", True))

    def setUseFullyConnectedPass(self, value: bool) -> None:
        self._op.graph.hints.setdefault("fc_pass", {})[self._op.uid] = bool(value)


def _pb_op(op: "Op") -> _PbOp:
    name = op.opdef.name
    if name == "repeat":
        return _PbLoopOp(op)
    if name == "call":
        return _PbCallOp(op)
    if name in ("matmul", "linear_bias_act", "matmul_pow2scaled"):
        return _PbMatMulOp(op)
    return _PbOp(op)


class _PbGraph:
    def __init__(self, graph: "Graph"):
        self._graph = graph
        self.id = graph.id

    def getOps(self):
        return [_pb_op(op) for op in self._graph.ops]

    def getOpSchedule(self, *_args, **_kwargs):
        """Ops run in the order they were recorded."""
        return self.getOps()

    def getCalledGraphs(self):
        seen, out = set(), []
        for op in self._graph.ops:
            callee = op.attrs.get("graph")
            if isinstance(callee, Graph) and id(callee) not in seen:
                seen.add(id(callee))
                out.append(_PbGraph(callee))
        return out

    def getInputIds(self):
        return [t.id for t in self._graph.inputs]

    def getOutputIds(self):
        return [t.id for t in self._graph.outputs]

    def __eq__(self, other):
        return isinstance(other, _PbGraph) and other._graph is self._graph

    def __hash__(self):
        return hash(id(self._graph))


class _RecordedOptions:
    """Session options of the reference substrate are IPU compiler / engine settings. Programs set them through
    attribute and item assignment (`opts.numIOTiles = 64`, `opts.engineOptions["x"] = "y"`,
    `opts.replicatedCollectivesSettings.prepareScheduleForMergingCollectives = True`); every such assignment is accepted
    and recorded, none changes what runs."""

    def __init__(self):
        object.__setattr__(self, "_values", {})

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return self._values.setdefault(name, _RecordedOptions())

    def __setattr__(self, name, value):
        self._values[name] = value

    def __getitem__(self, key):
        return self._values.setdefault(key, _RecordedOptions())

    def __setitem__(self, key, value):
        self._values[key] = value

    def __contains__(self, key):
        return key in self._values

    def __repr__(self):
        return f"Options({self._values})"


class _PbIrShim:
    """Minimal stand-in for the handful of low-level IR queries that user scripts written for the reference make."""

    def __init__(self, ir):
        self._ir = ir
        self._options = _RecordedOptions()

    def getAllGraphs(self):
        return [g._pb_graph for g in self._ir.graphs]

    def getSessionOptions(self):
        return self._options

    def setPatterns(self, patterns) -> None:
        """Accepted for scripts that configure popart's pattern sets by hand; the rewrite passes of this substrate are
        fixed (`applyPreAliasPatterns`)."""
        self._patterns = patterns

    def applyPreAliasPatterns(self, graph) -> int:
        from ..patterns import apply_patterns_to_graph

        return apply_patterns_to_graph(graph._graph if isinstance(graph, _PbGraph) else graph)

    def applyInplacePattern(self, graph) -> None:
        """Buffers are reused by the allocator, not by rewriting ops: nothing to do."""

    def logIr(self):
        for g in self._ir.graphs:
            print(f"--- {g.name}\n{g.print_ops()}")


class Ir:
    """Container of all graphs of one program plus the replication setup.

    `replication="popdist"` (or "distributed") takes the replica count from `torch.distributed` / the launcher
    environment: one replica per process, one process per GPU.
    """

    def __init__(self, replication: Union[int, str] = 1, devices_per_replica: int = 1):
        """`devices_per_replica` > 1 with `replication="popdist"`: every replica spans that many processes / GPUs, one
        per device slot (`ipu(i)`, a pipeline stage); process `rank` hosts slot `rank % devices_per_replica` of
        replica `rank // devices_per_replica`."""
        self.devices_per_replica = int(devices_per_replica)
        self.graphs: List[Graph] = []
        self._graph_counter = itertools.count()
        self._op_ids = itertools.count(100)
        self.main_graph = Graph(self, "main")
        self.graphs.append(self.main_graph)
        self.distributed = False
        if isinstance(replication, str):
            import os

            self.distributed = True
            world = int(os.environ.get("WORLD_SIZE", "1"))
            if world % self.devices_per_replica:
                raise ValueError(f"WORLD_SIZE={world} is not a multiple of devices_per_replica={devices_per_replica}")
            self._replication_factor = world // self.devices_per_replica
        else:
            self._replication_factor = int(replication)
        self.num_host_transfers = 1
        self.num_device_transfers = 1
        self._pb_ir = _PbIrShim(self)
        self.initial_values: Dict[Variable, Any] = {}
        self.remote_buffers: List[Any] = []
        self.streams: List[Any] = []
        self.options: Options = Options.from_env()

    # -- replication ----------------------------------------------------------------------------------------------
    @property
    def replication_factor(self) -> int:
        return self._replication_factor

    @replication_factor.setter
    def replication_factor(self, n: int):
        self._replication_factor = int(n)

    @property
    def instance_replication_factor(self) -> int:
        """Replicas hosted by this process: all of them in single-process simulation, one when launched one process
        per GPU."""
        return 1 if self.distributed else self._replication_factor

    def replica_grouping(self, stride: int = 1, group_size: Optional[int] = None) -> ReplicaGrouping:
        return ReplicaGrouping(self._replication_factor, stride, group_size)

    def replica_grouping_from_assignments(self, assignment: Sequence[int]) -> ReplicaGrouping:
        return ReplicaGrouping(self._replication_factor, assignment=assignment)

    # -- graph creation -------------------------------------------------------------------------------------------
    def _new_graph_name(self, base: str) -> str:
        return f"{base}_subgraph({next(self._graph_counter)})"

    def create_empty_graph(self, name: Optional[str] = None) -> Graph:
        g = Graph(self, self._new_graph_name(name or "graph"))
        self.graphs.append(g)
        return g

    def create_graph(self, fn: Callable, *args, **kwargs) -> Graph:
        """Trace `fn` into a new graph. Tensor / TensorSpec arguments (also inside lists) become graph inputs of the
        same spec; anything else is passed through unchanged. The returned tensors become the graph outputs."""
        if hasattr(fn, "build") and not inspect.isfunction(fn) and not inspect.ismethod(fn):
            base = type(fn).__name__
            sig_target = fn.build
        else:
            base = getattr(fn, "__name__", type(fn).__name__)
            sig_target = fn
        try:
            sig = inspect.signature(sig_target)
            bound = sig.bind(*args, **kwargs)
        except TypeError as e:
            raise ValueError(
                f"The arguments, {args} and {kwargs}, do not match the signature of the function {base}: {e}"
            ) from None
        g = self.create_empty_graph(base)
        new_args: List[Any] = []
        new_kwargs: Dict[str, Any] = {}

        def convert(value, pname, by_ref):
            if isinstance(value, (Tensor, TensorSpec)):
                ref = by_ref or (isinstance(value, Tensor) and value.graph.is_by_ref(value) and False)
                return graph_input(value.shape, value.dtype, pname, by_ref=ref, meta_shape=value.meta_shape)
            if isinstance(value, (list, tuple)) and value and all(isinstance(v, (Tensor, TensorSpec)) for v in value):
                return type(value)(convert(v, f"{pname}_{i}", by_ref) for i, v in enumerate(value))
            return value

        with g:
            for pname, value in bound.arguments.items():
                param = sig.parameters[pname]
                ann = param.annotation
                by_ref = ann is TensorByRef or "TensorByRef" in str(ann)
                if param.kind == inspect.Parameter.VAR_POSITIONAL:
                    new_args.extend(convert(v, f"{pname}_{i}", by_ref) for i, v in enumerate(value))
                elif param.kind == inspect.Parameter.VAR_KEYWORD:
                    for k, v in value.items():
                        new_kwargs[k] = convert(v, k, by_ref)
                elif param.kind == inspect.Parameter.KEYWORD_ONLY or pname in kwargs:
                    # given by keyword: passed on by keyword (a defaulted parameter before it may have been left out)
                    new_kwargs[pname] = convert(value, pname, by_ref)
                else:
                    new_args.append(convert(value, pname, by_ref))
            result = fn(*new_args, **new_kwargs)
            if result is None:
                result = ()
            elif isinstance(result, Tensor):
                result = (result,)
            for out in result:
                if not isinstance(out, Tensor):
                    raise ValueError(f"Graph outputs must be tensors, got {type(out)} from {base}")
                graph_output(out)
        return g

    def _next_op_id(self) -> int:
        return next(self._op_ids)

    def get_all_h2d_streams(self) -> List[Any]:
        from .buffers import HostToDeviceStream

        return [st for st in self.streams if isinstance(st, HostToDeviceStream)]

    def get_all_d2h_streams(self) -> List[Any]:
        from .buffers import DeviceToHostStream

        return [st for st in self.streams if isinstance(st, DeviceToHostStream)]

    @property
    def num_device_iterations(self) -> int:
        """Host transfers per `Session.run` (the name newer popxl releases use for `num_host_transfers`)."""
        return self.num_host_transfers

    @num_device_iterations.setter
    def num_device_iterations(self, n: int):
        self.num_host_transfers = int(n)

    def dot_checkpoint(self, check: str = "") -> None:
        """The reference substrate dumps a Graphviz file of the IR here when asked to through an environment variable;
        `ir._pb_ir.logIr()` prints this substrate's graphs instead."""

    def __repr__(self):
        return f"Ir(graphs={len(self.graphs)}, replication_factor={self._replication_factor})"


# ---------------------------------------------------------------------------------------------------------------
# lazily materialised initial values
# ---------------------------------------------------------------------------------------------------------------


class LazyInit:
    """Initial value of a variable described by a recipe instead of a host array. It is materialised directly on the
    session's device (per replica group, seeded by `seed + group index`), so a multi-billion-parameter model neither
    needs host memory for its initial weights nor a host-to-device copy of them.
    `kind`: "normal" (mean 0, `std`), "zeros", "ones", or "copy" (value of variable `source`, cast)."""

    def __init__(self, shape, dtype=np.float32, kind: str = "normal", std: float = 0.02, seed: int = 0, source=None,
                 groups: int = 0):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype) if not isinstance(dtype, _dt.dtype) else dtype
        self.kind, self.std, self.seed, self.source, self.groups = kind, std, seed, source, groups
        self.ndim = len(self.shape)

    def with_groups(self, n: int) -> "LazyInit":
        """Same recipe for `n` replica groups (host shape gains a leading axis of `n`)."""
        out = LazyInit((n, *self.shape), self.dtype, self.kind, self.std, self.seed, self.source, groups=n)
        return out

    def astype(self, dtype):
        return LazyInit(self.shape, dtype, self.kind, self.std, self.seed, self.source, self.groups)

    def materialize(self, device, torch_dtype, group: int = 0) -> torch.Tensor:
        shape = self.shape[1:] if self.groups else self.shape
        if self.kind == "zeros":
            return torch.zeros(shape, dtype=torch_dtype, device=device)
        if self.kind == "ones":
            return torch.ones(shape, dtype=torch_dtype, device=device)
        if self.kind == "normal":
            gen = torch.Generator(device=device)
            gen.manual_seed((self.seed + 7919 * group) & 0x7FFFFFFF)
            # always drawn in fp32 so that a 16-bit weight and its fp32 master copy (same recipe) agree exactly
            t = torch.empty(shape, dtype=torch.float32, device=device)
            t.normal_(0.0, self.std, generator=gen)
            return t.to(torch_dtype)
        raise ValueError(f"LazyInit kind {self.kind!r} cannot be materialised on its own")


# ---------------------------------------------------------------------------------------------------------------
# tensor factories
# ---------------------------------------------------------------------------------------------------------------


def graph_input(shape: Iterable[int], dtype: dtype, name: Optional[str] = None, by_ref: bool = False,
                meta_shape: Optional[Iterable[int]] = None) -> Tensor:
    g = gcg()
    t = Tensor(g, shape, dtype, name or "input", meta_shape)
    t.kind = "input"
    g._inputs.append(t)
    if by_ref:
        g._by_ref.add(t)
    return t


def graph_output(t: Tensor) -> None:
    g = gcg()
    if t.graph is not g:
        raise ValueError(f"{t} is not in the current graph {g.name}")
    g._outputs.append(t)


def _host_array(data, dt: Optional[dtype]):
    if isinstance(data, LazyInit):
        return data
    if isinstance(data, torch.Tensor):
        t = data.detach().cpu()
    else:
        arr = np.asarray(data)
        if dt is None and arr.dtype == np.float64:
            arr = arr.astype(np.float32)
        if dt is None and arr.dtype == np.int64:
            arr = arr.astype(np.int32)
        t = _dt.to_torch(arr)
    if dt is not None and t.dtype != dt.as_torch():
        t = t.to(dt.as_torch())
    return t


def variable(data, dtype: Optional[dtype] = None, name: Optional[str] = None, downcast: bool = True,
             replica_grouping: Optional[ReplicaGrouping] = None, retrieval_mode=None, log2_scale=None,
             nan_on_overflow=None) -> Variable:
    """Create a variable in the main graph initialised with `data` (host shape: `(num_groups, *shape)` when the
    replica grouping has more than one group)."""
    g = gcg()
    if g is not g.ir.main_graph:
        raise ValueError("Variables can only be created in the main graph")
    dt = _dt.dtype.as_dtype(dtype) if dtype is not None else None
    host = data if isinstance(data, np.memmap) else _host_array(data, dt)
    if isinstance(host, (np.memmap, LazyInit)):
        dt = dt or _dt.dtype.as_dtype(host.dtype)
        full_shape = tuple(host.shape)
    else:
        dt = _dt.dtype.as_dtype(host.dtype)
        full_shape = tuple(host.shape)
    rg = replica_grouping or g.ir.replica_grouping()
    if rg.num_groups > 1:
        if not full_shape or full_shape[0] != rg.num_groups:
            raise ValueError(
                f"Variable data for a replica grouping with {rg.num_groups} groups must have a leading axis of that "
                f"size. Got shape {full_shape}")
        shape = full_shape[1:]
    else:
        shape = full_shape
    v = Variable(g, shape, dt, name or "variable", replica_grouping=rg)
    g.ir.initial_values[v] = host
    if isinstance(host, np.memmap):
        v._memmap_arr = host
    return v


def constant(data, dtype: Optional[dtype] = None, name: Optional[str] = None, downcast: bool = True) -> Constant:
    g = gcg()
    dt = _dt.dtype.as_dtype(dtype) if dtype is not None else None
    return Constant(g, _host_array(data, dt), name or "const")


def replica_sharded_variable(data, dtype: Optional[dtype] = None, name: Optional[str] = None,
                             replica_grouping: Optional[ReplicaGrouping] = None,
                             shard_over: Optional[int] = None, shard_grouping=None):
    """Variable stored as flat `1/shard_over` shards. Returns `(variable, shard_tensor)`; here the variable *is* the
    per-replica shard, so both entries are the same tensor."""
    g = gcg()
    dt = _dt.dtype.as_dtype(dtype) if dtype is not None else None
    host = _host_array(data, dt)
    rg = replica_grouping or g.ir.replica_grouping()
    full_shape = tuple(host.shape[1:]) if rg.num_groups > 1 else tuple(host.shape)
    if shard_grouping is None:
        shard_over = shard_over or rg.group_size
        shard_grouping = _shard_grouping_within(rg, shard_over)
    nelms = int(np.prod(full_shape)) if full_shape else 1
    n = shard_grouping.group_size
    if nelms % n != 0:
        raise ValueError(f"Cannot shard {nelms} elements over {n} replicas")
    v = Variable(g, (nelms // n,), dt or _dt.dtype.as_dtype(host.dtype), name or "variable", meta_shape=full_shape,
                 replica_grouping=rg, shard_group=shard_grouping)
    g.ir.initial_values[v] = host
    return v, v


def _shard_grouping_within(rg: ReplicaGrouping, shard_over: int) -> ReplicaGrouping:
    """Sub-grouping of `rg` with `shard_over` members per group (the first `shard_over` positions, then the next...)."""
    if shard_over == rg.group_size:
        return rg
    if rg.group_size % shard_over != 0:
        raise ValueError(f"shard_over={shard_over} must divide the group size {rg.group_size}")
    assign = [0] * rg.num_replicas
    per = rg.group_size // shard_over
    for gi, members in enumerate(rg.groups):
        for pos, r in enumerate(members):
            assign[r] = gi * per + pos // shard_over
    return ReplicaGrouping(rg.num_replicas, assignment=assign)
