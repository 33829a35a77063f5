"""Import path kept for parity with popxl_addons/ops/replicated_strided_collectives/replicated_all_gather_strided.py."""
from . import *  # noqa: F401,F403
from . import __all__  # noqa: F401
