"""popxl_addons_b200: the popxl.addons programming model (modules -> graphs + variable factories, explicit gradient
graphs, execution-scheme transforms, replica groupings with tensor sharding) on PyTorch tensors and hand-written
sm_100a CUDA kernels, one process per GPU.

`import popxl_addons_b200 as addons`; the graph substrate is `addons.xl` (use it where reference code says `popxl`).
Top-level names follow popxl_addons/__init__.py:2-15.
"""
from . import xl
from .module import *  # noqa: F401,F403
from .module import Module, NameScopeMeta, create_grad_graph_info
from .graph_cache import *  # noqa: F401,F403
from .remote import *  # noqa: F401,F403
from .route_tensor import *  # noqa: F401,F403
from .ops import *  # noqa: F401,F403
from .transforms import *  # noqa: F401,F403
from .seed_variable import *  # noqa: F401,F403
from .streams import *  # noqa: F401,F403
from .utils import *  # noqa: F401,F403
from .task_session import *  # noqa: F401,F403
from .performance_utils import *  # noqa: F401,F403
from .debugging import *  # noqa: F401,F403
from .array_munging import *  # noqa: F401,F403
from . import layers, ops, optimizers, transforms  # noqa: F401


def _git_commit() -> str:
    import os
    import subprocess

    try:
        here = os.path.dirname(os.path.abspath(__file__))
        return subprocess.check_output(["git", "rev-parse", "HEAD"], cwd=here, stderr=subprocess.DEVNULL,
                                       timeout=5).decode().strip()
    except Exception:
        return "unknown"


GIT_COMMIT = _git_commit()
__version__ = "0.1.0"
