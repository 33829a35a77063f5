"""Graph transforms. Parity: popxl_addons/transforms/__init__.py:2-7."""
from .autodiff import autodiff, autodiff_with_accumulation, remap_grad_info
from .available_memory_proportion import (set_available_memory_proportion_by_ipu,
                                          set_graph_available_memory_proportion_by_ipu)
from .batch_serialisation import (batch_serialise, batch_serialise_fwd_and_grad, batch_serial_buffer, RemoteHandle)
from .pipelining import pipelined_execution
from .recomputation import recompute_graph, add_recompute_inputs
from .use_fc_pass import disable_fc_pass, enable_fc_pass
