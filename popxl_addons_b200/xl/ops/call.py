"""`xl.ops.call` (popxl/ops/call.py)."""
from .control import CallSiteInfo, call, call_with_info  # noqa: F401

__all__ = ["call", "call_with_info", "CallSiteInfo"]
