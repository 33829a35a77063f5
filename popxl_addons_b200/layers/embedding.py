"""Embedding lookup, optionally with the vocabulary sharded across a tensor-parallel group.

When sharded, every replica holds `ceil(vocab / n)` rows rounded up to a multiple of 16; the caller subtracts the
replica's row offset from the token ids, rows outside the local shard come back as zeros and the partial results are
summed by the tensor-parallel all-reduce that follows.
Parity: popxl_addons/layers/embedding.py:17-79.
"""
import math
from functools import partial
from typing import Dict, Optional

import numpy as np

from .. import xl
from ..module import Module
from ..named_tensors import NamedTensors
from ..xl import ops
from .linear import truncnorm_init

__all__ = ["Embedding"]

_SHARD_MULTIPLE = 16


def model_vocab_shard_size(vocab_size: int, n_shards: int) -> int:
    """Rows per vocabulary shard in the decoder models of this package: padded to a multiple of 16 only when the
    vocabulary is actually sharded."""
    if n_shards <= 1:
        return vocab_size
    return Embedding.get_vocab_shard_size(vocab_size, n_shards)


def model_vocab_offsets(vocab_size: int, n_shards: int) -> np.ndarray:
    return np.arange(n_shards, dtype=np.int64) * model_vocab_shard_size(vocab_size, n_shards)


class Embedding(Module):
    def __init__(self, dtype: xl.dtype, vocab_size: int, hidden_size: int, axis: int = 0,
                 replica_grouping: Optional[xl.ReplicaGrouping] = None):
        super().__init__()
        self.dtype = dtype
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.axis = axis
        self.replica_grouping = replica_grouping
        self.n_shards = replica_grouping.num_groups if replica_grouping is not None else 1
        self.vocab_shard_size = self.get_vocab_shard_size(vocab_size, self.n_shards)
        self.offsets = self.get_offsets(vocab_size, self.n_shards)

    @staticmethod
    def get_vocab_shard_size(vocab_size: int, n_shards: int) -> int:
        """Rows per shard: `ceil(vocab_size / n_shards)` rounded up to a multiple of 16, also for a single shard (the
        reference's rule, popxl_addons/layers/embedding.py:48-52: a checkpoint of its embedding has that many rows)."""
        return _SHARD_MULTIPLE * math.ceil(math.ceil(vocab_size / n_shards) / _SHARD_MULTIPLE)

    @staticmethod
    def get_offsets(vocab_size: int, n_shards: int) -> np.ndarray:
        """First vocabulary row of every shard."""
        return np.arange(n_shards, dtype=np.int64) * Embedding.get_vocab_shard_size(vocab_size, n_shards)

    @staticmethod
    def get_padded_size(vocab_size: int, n_shards: int) -> int:
        return n_shards * Embedding.get_vocab_shard_size(vocab_size, n_shards)

    def build(self, indices: xl.Tensor) -> xl.Tensor:
        """`indices` must already have this shard's offset subtracted when the vocabulary is sharded."""
        np_dt = self.dtype.as_numpy() if self.dtype._numpy is not None else np.float32
        shape = (self.vocab_shard_size, self.hidden_size)
        w = self.add_variable_input("weight", partial(truncnorm_init, shape, 0.02, np_dt), self.dtype,
                                    replica_grouping=self.replica_grouping)
        return ops.gather(w, indices, axis=self.axis, zero_OOR=self.n_shards > 1)

    @staticmethod
    def torch_mapping(variables: NamedTensors, nn_layer, n_shards: int = 1) -> Dict[xl.Tensor, np.ndarray]:
        """Pads the vocabulary to `n_shards * shard_size` rows and splits it into a leading shard axis."""
        w = nn_layer.weight.data.detach().cpu().numpy()
        size = Embedding.get_vocab_shard_size(w.shape[0], n_shards)
        w = np.pad(w, ((0, size * n_shards - w.shape[0]), (0, 0)))
        if n_shards > 1:
            w = w.reshape(n_shards, size, w.shape[1])
        return {variables.weight: w.copy()}
