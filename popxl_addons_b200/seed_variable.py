"""Random seed held in a variable, so it is checkpointed and identical within each replica group.
Parity: popxl_addons/seed_variable.py:13-33."""
from typing import Optional, Tuple

import numpy as np

from . import xl

__all__ = ["seed_variable"]


def seed_variable(seed: int, replica_grouping: Optional[xl.ReplicaGrouping] = None) -> Tuple[xl.Variable, xl.Tensor]:
    """Returns `(variable, tensor to use in the graph)`. Each replica group gets its own seed pair derived from
    `seed` (shape `(2,)` uint32); replicas inside a group share it."""
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping()
    rng = np.random.Generator(np.random.PCG64(seed))
    data = rng.integers(0, 2 ** 32, size=(rg.num_groups, 2), dtype=np.uint64).astype(np.uint32)
    if rg.num_groups == 1:
        data = data[0]
    with ir.main_graph:
        var = xl.variable(data, xl.uint32, "seed", replica_grouping=rg)
    return var, var
