"""Add-on ops. Only the light, pure-graph ops are imported here; ops backed by native CUDA kernels live in their own
modules and are imported by path (`from popxl_addons_b200.ops.rotary_pos_embed import rotary_pos_embed`), so importing
the package never needs the compiled extension.

Parity: popxl_addons/ops/__init__.py:3-5.
"""
from .cross_entropy import cross_entropy, cross_entropy_with_grad
from .streams import host_load, host_store
from .fp8_amax_scale import fp8_amax_scale

__all__ = ["cross_entropy", "cross_entropy_with_grad", "host_load", "host_store", "fp8_amax_scale"]
