"""Multi-GPU runtime: symmetric-memory arenas over NVLink / NVSwitch, the fused compute + collective kernels that use
them, and the graph pass that rewrites GEMM -> all-reduce pairs into one fused op."""
from .passes import (fuse_gemm_collectives, fuse_matmul_sums, fuse_sequence_parallel_collectives,
                     schedule_collective_overlap)

__all__ = ["fuse_gemm_collectives", "fuse_matmul_sums", "fuse_sequence_parallel_collectives",
           "schedule_collective_overlap"]
