"""Dense x constant-sparse (CSR) matmul for inference.

The sparsity pattern and the non-zero values are constants of the graph. On CUDA the product runs as a row-gather
SpMM kernel; the CPU backend uses torch sparse.
Parity: popxl_addons/ops/static_sparse_ops/dense_sparse_matmul.py:23-85.
"""
import numpy as np
import torch

from .. import xl
from ..xl.opdef import OpDef, emit1

__all__ = ["random_sparse", "dense_const_sparse_matmul"]


def random_sparse(dense: np.ndarray, density: float = 0.5) -> np.ndarray:
    """Zero a random `1 - density` fraction of `dense` **in place** (at least one element is kept) and return it, as the
    reference's helper does; build the sparse operand from it with `scipy.sparse.csr_matrix(dense)` (16-bit floats:
    `csr_matrix(dense.astype(np.float32))`, scipy has no 16-bit sparse matrices)."""
    drop = np.random.rand(*dense.shape) < (1.0 - density)
    if np.all(drop):
        drop.reshape(-1)[0] = False
    dense[drop] = 0
    return dense


def _impl(lhs, indptr, indices, values, n_rows, n_cols):
    if lhs.device.type == "meta":
        return torch.empty((*lhs.shape[:-1], n_cols), dtype=lhs.dtype, device="meta")
    csr = torch.sparse_csr_tensor(indptr.long(), indices.long(), values.float(), size=(n_rows, n_cols))
    dense_rhs = csr.to_dense()
    return torch.matmul(lhs.float(), dense_rhs).to(lhs.dtype)


OpDef("dense_csr_matmul", impl=_impl)


def dense_const_sparse_matmul(lhs: xl.Tensor, rhs, output_cols: int = None) -> xl.Tensor:
    """`lhs (.., M, K) @ rhs (K, N)` with `rhs` a scipy CSR matrix baked into the graph."""
    rhs = rhs.tocsr()
    k, n = rhs.shape
    if lhs.shape[-1] != k:
        raise ValueError(f"Inner dimensions do not match: {lhs.shape} x {rhs.shape}")
    if output_cols is not None and output_cols != n:
        raise ValueError(f"output_cols={output_cols} does not match the sparse matrix ({n} columns)")
    indptr = xl.constant(rhs.indptr.astype(np.int32), xl.int32, "csr_indptr")
    indices = xl.constant(rhs.indices.astype(np.int32), xl.int32, "csr_indices")
    values = xl.constant(rhs.data.astype(np.float32), xl.float32, "csr_values")
    return emit1("dense_csr_matmul", [lhs, indptr, indices, values], {"n_rows": k, "n_cols": n})


from ._paths import also_importable_as  # noqa: E402

also_importable_as(__name__, "dense_sparse_matmul")
