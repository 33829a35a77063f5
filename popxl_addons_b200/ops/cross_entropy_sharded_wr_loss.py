"""Vocabulary-sharded cross-entropy over the device slots of one replica, under the reference's module path
(popxl_addons/ops/cross_entropy_sharded_wr_loss/cross_entropy_sharded_wr_loss.py:40-89). The op is defined beside its
across-replica sibling."""
from .cross_entropy_sharded_loss import cross_entropy_sharded_wr_loss

__all__ = ["cross_entropy_sharded_wr_loss"]


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__)
