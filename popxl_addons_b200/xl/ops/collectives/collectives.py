"""`xl.ops.collectives.collectives` (popxl/ops/collectives/collectives.py): the names of the reduction operators."""
import enum
from typing import Union

try:
    from typing import Literal
except ImportError:  # pragma: no cover
    from typing_extensions import Literal

__all__ = ["CollectiveOps", "CollectiveOperator", "to_collective_op"]

CollectiveOps = Literal["add", "mean", "mul", "min", "max", "logical_and", "logical_or", "square_add", "local"]


class CollectiveOperator(enum.Enum):
    Add = "add"
    Mean = "mean"
    Mul = "mul"
    Min = "min"
    Max = "max"
    LogicalAnd = "logical_and"
    LogicalOr = "logical_or"
    SquareAdd = "square_add"
    Local = "local"

    @property
    def name_(self) -> str:
        return self.value


def to_collective_op(op: Union[str, CollectiveOperator]) -> CollectiveOperator:
    """`"add"` / `CollectiveOperator.Add` -> the operator; unknown names raise ValueError. Ops of this substrate
    take either form (and reduce with `add`, `mean`, `max`, `min` or `mul`)."""
    if isinstance(op, CollectiveOperator):
        return op
    try:
        return CollectiveOperator(str(op).lower())
    except ValueError:
        raise ValueError(f"Not a valid op: {op}. Must choose from: {', '.join(o.value for o in CollectiveOperator)}") \
            from None
