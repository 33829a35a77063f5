"""`xl.tensor`: the tensor classes and their constructors under popxl's module path (popxl/tensor.py)."""
from typing import Union

import numpy as np
import torch

from .core import (Constant, Tensor, TensorByRef, TensorSpec, Variable, constant, graph_input, graph_output,  # noqa: F401
                   replica_sharded_variable, variable)
from .buffers import remote_replica_sharded_variable, remote_variable  # noqa: F401

# what `variable(...)`, `constant(...)` and the session accept as host data
host_tensor_types = (np.ndarray, torch.Tensor)
HostTensor = Union[np.ndarray, torch.Tensor]
HostScalarTensor = Union[int, float, bool, HostTensor]
TensorLike = Union[Tensor, HostScalarTensor]

__all__ = ["Tensor", "Variable", "Constant", "TensorByRef", "TensorSpec", "HostTensor", "HostScalarTensor", "TensorLike",
           "host_tensor_types", "variable", "constant", "graph_input", "graph_output", "replica_sharded_variable",
           "remote_variable", "remote_replica_sharded_variable"]
