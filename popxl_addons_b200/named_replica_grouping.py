"""Named replica groupings and helpers that restrict a grouping to one process or to one NVSwitch domain.

The reference distinguishes replicas of one *instance* (process) and of one *IPU-link domain*; the analogues here are
"replicas hosted by this process" and "ranks of one NVSwitch domain (node)", whose size comes from the environment
variable `XL_NVLINK_DOMAIN_SIZE` (default: `min(replication_factor, 8)`).

Parity: popxl_addons/named_replica_grouping.py:20-107.
"""
import os
from typing import Iterable, Optional

from . import xl
from .dot_tree import DotTree

__all__ = ["NamedReplicaGrouping", "get_instance_replica_grouping", "is_cross_instance", "get_ild_size_from_popdist",
           "get_ild_replica_grouping", "is_cross_ild", "fill_none_group"]


class NamedReplicaGrouping(DotTree):
    @classmethod
    def build_groups(cls, names: Iterable[str], value: xl.ReplicaGrouping) -> "NamedReplicaGrouping":
        """Same grouping under every name."""
        return cls.from_dict({n: value for n in names})


def fill_none_group(rg: Optional[xl.ReplicaGrouping], none_value: xl.ReplicaGrouping) -> xl.ReplicaGrouping:
    return none_value if rg is None else rg


def _restrict(rg: xl.ReplicaGrouping, domain: int) -> xl.ReplicaGrouping:
    """Grouping over `domain` consecutive replicas whose groups are `rg`'s groups intersected with the domain."""
    ir_n = rg.num_replicas
    if domain >= ir_n:
        return rg
    assign = rg.assignment[:domain]
    remap = {}
    local = [remap.setdefault(a, len(remap)) for a in assign]
    return xl.ReplicaGrouping(domain, assignment=local)


def get_instance_replica_grouping(replica_grouping: Optional[xl.ReplicaGrouping] = None) -> xl.ReplicaGrouping:
    """The part of a grouping that lies within the replicas hosted by one process."""
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping()
    return _restrict(rg, ir.instance_replication_factor)


def is_cross_instance(replica_grouping: Optional[xl.ReplicaGrouping] = None) -> bool:
    """Does any group span more than one process?"""
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping()
    n = ir.instance_replication_factor
    return any(len({r // n for r in members}) > 1 for members in rg.groups)


def get_ild_size_from_popdist() -> int:
    """Ranks per NVSwitch domain."""
    rf = xl.gcg().ir.replication_factor
    return int(os.environ.get("XL_NVLINK_DOMAIN_SIZE", min(rf, 8)))


def get_ild_replica_grouping(replica_grouping: Optional[xl.ReplicaGrouping] = None) -> xl.ReplicaGrouping:
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping()
    return _restrict(rg, get_ild_size_from_popdist())


def is_cross_ild(replica_grouping: Optional[xl.ReplicaGrouping] = None) -> bool:
    """Does any group span more than one NVSwitch domain (i.e. need the inter-node network)?"""
    ir = xl.gcg().ir
    rg = replica_grouping or ir.replica_grouping()
    n = get_ild_size_from_popdist()
    return any(len({r // n for r in members}) > 1 for members in rg.groups)
