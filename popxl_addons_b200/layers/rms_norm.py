"""RMSNorm (Llama-style) over the last axis. No reference counterpart; needed by the Llama configuration."""
from functools import partial

import numpy as np

from .. import xl
from ..module import Module
from ..xl import ops

__all__ = ["RMSNorm"]


class RMSNorm(Module):
    def __init__(self, eps: float = 1e-5):
        super().__init__()
        self.eps = eps

    def build(self, x: xl.Tensor) -> xl.Tensor:
        np_dt = x.dtype.as_numpy() if x.dtype._numpy is not None else np.float32
        w = self.add_variable_input("weight", partial(np.ones, x.shape[-1], np_dt), x.dtype)
        return ops.rms_norm(x, w, eps=self.eps)
