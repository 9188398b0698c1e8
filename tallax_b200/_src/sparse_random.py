"""Counter-based noise at arbitrary positions (mirror of tallax/_src/sparse_random.py:43-94)."""
from __future__ import annotations

import torch

from tallax_b200._src import ops

F32_TINY = 1.1754943508222875e-38


def sparse_random_uniform(key_ref, indices, dim1_size, dtype=torch.float32, minval=0.0, maxval=1.0):
    """Uniform noise equal to the dense jax.random.uniform(key, (*, dim1_size)) read at
    (indices[0], indices[1]): threefry2x32 with counter (0, i0 * dim1_size + i1)."""
    assert len(indices) == 2
    if dtype != torch.float32:
        raise NotImplementedError
    return ops.sparse_random_uniform(key_ref, indices[0], indices[1], dim1_size, minval, maxval)


def sparse_random_categorical(key_ref, logits, indices, dim1_size, axis=-1, dtype=torch.float32):
    """Gumbel arg-max over `logits` with noise indexed by `indices`; returns the winning
    entry of every index array along `axis` (sparse_random.py:68-94)."""
    if dtype != torch.float32:
        raise NotImplementedError
    axis = axis if axis >= 0 else logits.ndim + axis
    return ops.gumbel_argmax(key_ref, logits, indices[0], indices[1], dim1_size, axis)
