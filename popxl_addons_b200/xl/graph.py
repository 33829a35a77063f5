"""`xl.graph` (popxl/graph.py)."""
from .core import Graph  # noqa: F401

__all__ = ["Graph"]
