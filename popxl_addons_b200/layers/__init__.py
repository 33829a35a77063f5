"""Layers. Those backed by native-only ops are imported by path (e.g. `layers.linear_gq.LinearGQ`).
Parity: popxl_addons/layers/__init__.py:3-8."""
from .linear import Linear
from .layer_norm import LayerNorm
from .group_norm import GroupNorm
from .embedding import Embedding
from .conv import Conv2D

__all__ = ["Linear", "LayerNorm", "GroupNorm", "Embedding", "Conv2D"]
