"""Random seed held in a variable, so it is checkpointed and identical within each replica group.
Parity: popxl_addons/seed_variable.py:13-33."""
from typing import Optional, Tuple

from . import xl

__all__ = ["seed_variable"]


def seed_variable(seed: int, replica_grouping: Optional[xl.ReplicaGrouping] = None) -> Tuple[xl.Variable, xl.Tensor]:
    """Returns `(variable, tensor to use in the graph)`. Each replica group gets its own seed pair derived from
    `seed` (shape `(2,)` uint32); replicas inside a group share it. Without a grouping every replica draws its own
    (groups of one replica, as in the reference)."""
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping(group_size=1)
    data = xl.create_seeds(seed, replicas=rg.num_groups)
    with ir.main_graph:
        var = xl.variable(data, xl.uint32, "seed", replica_grouping=rg)
    return var, var
