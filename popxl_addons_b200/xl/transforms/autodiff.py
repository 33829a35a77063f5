"""`xl.transforms.autodiff` as a module path (popxl/transforms/autodiff.py): the transform and its result types."""
from ..autodiff import ExpectedConnection, ExpectedConnectionType, GradGraphInfo, autodiff  # noqa: F401

__all__ = ["autodiff", "GradGraphInfo", "ExpectedConnection", "ExpectedConnectionType"]
