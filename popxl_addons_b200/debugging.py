"""Device-side prints gated by the environment variable `MODEL_LOG_LEVEL` (TRACE < DEBUG < INFO < WARN).
Parity: popxl_addons/debugging.py:14-45."""
import os
from typing import Optional

from . import xl
from .xl import ops

__all__ = ["print_tensor", "print_text", "check_run_to_run_determinism"]

_LEVELS = {"TRACE": 0, "DEBUG": 1, "INFO": 2, "WARN": 3, "OFF": 4}


def _enabled(level: str) -> bool:
    if level not in _LEVELS:
        raise ValueError(f"level must be one of {list(_LEVELS)}. Not: {level}")
    current = os.environ.get("MODEL_LOG_LEVEL", "OFF").upper()
    return _LEVELS.get(current, 4) <= _LEVELS[level]


def print_tensor(t: xl.Tensor, *args, level: str = "DEBUG", **kwargs) -> xl.Tensor:
    """`ops.print_tensor` when the log level allows it, else `t` unchanged."""
    return ops.print_tensor(t, *args, **kwargs) if _enabled(level) else t


def print_text(text: str, num: Optional[xl.Tensor] = None, level: str = "DEBUG"):
    """Print `text` at run time (a tensor is needed to anchor the print; a dummy constant is used if none given)."""
    if not _enabled(level):
        return num
    anchor = num if num is not None else xl.constant(0, xl.int32)
    return ops.print_tensor(anchor, title=text)


def check_run_to_run_determinism(session, inputs, runs: int = 2, variables=None):
    """Race detection without a sanitizer: run the program `runs` times from the same state and inputs and compare
    every output stream and every listed variable bit for bit. The kernels reduce in a fixed order, so a difference
    means unordered accesses (a missing dependency between streams, a buffer reused too early, a lost update of a
    by-reference input). Returns the list of names that differed (empty = deterministic); the session's state is
    restored to what it was before the call. The reference has no such tool (it relies on popart's topological
    constraints, popxl_addons/optimizers/adam.py:18)."""
    import numpy as np

    state = list(variables) if variables is not None else list(session.ir.initial_values)
    state = [v for v in state if getattr(v, "remote_buffer", None) is None and session.owns(v)]
    snapshot = session.get_tensors_data(state)
    results = []
    for _ in range(runs):
        session.write_variables_data(snapshot)
        out = session.run(inputs)
        after = session.get_tensors_data(state)
        results.append(({s.name: np.array(a, copy=True) for s, a in out.items()},
                        {v.name: np.array(a, copy=True) for v, a in after.items()}))
    session.write_variables_data(snapshot)
    differing = []
    for kind in (0, 1):
        for name, ref in results[0][kind].items():
            for other in results[1:]:
                a, b = ref, other[kind][name]
                if a.shape != b.shape or a.tobytes() != b.tobytes():
                    differing.append(name)
                    break
    return differing
