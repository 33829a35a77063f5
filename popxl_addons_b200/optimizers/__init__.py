from .adam import AdamOptimizerStep
from .sgd import SGDOptimizerStep

__all__ = ["AdamOptimizerStep", "SGDOptimizerStep"]
