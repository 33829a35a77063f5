"""Type aliases shared by the graph containers and the autodiff transform: what may stand for a graph, for the result
of autodiff, and for the map from called graphs to their gradient graphs. Parity: popxl_addons/graph_common.py:10-40."""
from typing import TYPE_CHECKING, Mapping, Optional, Tuple, Union

from . import xl
from .xl.autodiff import GradGraphInfo

if TYPE_CHECKING:  # pragma: no cover
    from .graph import BoundGraph, GraphWithNamedArgs

__all__ = ["GraphLike", "GradGraphInfoLike", "CalledGraphsGradInfoLike", "CalledGraphsGradInfo",
           "normalise_called_graphs_grad_info"]

GraphLike = Union[xl.Graph, "GraphWithNamedArgs", "BoundGraph"]
GradGraphInfoLike = Union[GradGraphInfo, "GraphWithNamedArgs"]
CalledGraphsGradInfoLike = Mapping[GraphLike, GradGraphInfoLike]
CalledGraphsGradInfo = Mapping[xl.Graph, GradGraphInfo]


def _pair(fwd_graph: GraphLike, grad_graph: GradGraphInfoLike) -> Tuple[xl.Graph, GradGraphInfo]:
    fwd = fwd_graph if isinstance(fwd_graph, xl.Graph) else fwd_graph.graph
    grad = grad_graph if isinstance(grad_graph, GradGraphInfo) else grad_graph.grad_graph_info
    return fwd, grad


def normalise_called_graphs_grad_info(called_graphs_grad_info: Optional[CalledGraphsGradInfoLike] = None
                                      ) -> CalledGraphsGradInfo:
    """`{graph-like: grad-info-like}` -> `{Graph: GradGraphInfo}` (wrappers are unwrapped, None gives `{}`)."""
    return dict(_pair(f, g) for f, g in (called_graphs_grad_info or {}).items())


_normalise_called_graphs_grad_info = _pair
_normalise_called_graphs_grad_info_dict = normalise_called_graphs_grad_info
