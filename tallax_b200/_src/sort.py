"""Multi-operand key/payload sort (mirror of tallax/_src/sort.py:768-929)."""
from __future__ import annotations

import torch

from tallax_b200._src import ops


def canonicalize_operand(operand):
    """utils.py:172-181: list of same-shape 2-D arrays."""
    operands = list(operand) if isinstance(operand, (list, tuple)) else [operand]
    shapes = [tuple(x.shape) for x in operands]
    if len(set(shapes)) != 1:
        raise ValueError(f"Inputs must all have the same shape, but found {shapes=}")
    if len(shapes[0]) != 2:
        raise ValueError("Only 2D inputs supported")
    return operands, shapes[0]


def _canonical_float(x):
    # what a key looks like after the key-domain round trip (-0 -> +0, canonical NaN): in place, by the
    # library's own kernel (x is the freshly gathered output)
    return ops.canonicalize_keys_(x)


def sort(operand, num_keys: int, is_stable: bool = False, return_argsort: bool = False, descending: bool = False,
         num_vmem_substages=None, block_token=None, interpret: bool = False):
    """Row-wise sort of one or several [rows, n] tensors.

    The first `num_keys` operands are lexicographic keys, the rest payloads.  The result
    is always the stable order (ties keep ascending column order, also when descending),
    which is a valid answer for the unstable variants too.  `num_vmem_substages`,
    `block_token` and `interpret` are TPU tuning knobs, accepted and ignored.
    """
    operands, shape = canonicalize_operand(operand)
    if not 1 <= num_keys <= len(operands):
        raise ValueError("num_keys must be between 1 and the number of operands")
    # least-significant key first; each pass is a stable argsort composed with the previous permutation
    perm = None
    sorted_first = None
    for j in reversed(range(num_keys)):
        want_keys = j == 0
        sorted_first, perm = ops.argsort_rows(operands[j], descending=descending, in_perm=perm, want_keys=want_keys)
    outs = []
    for i, x in enumerate(operands):
        if i == 0:
            outs.append(sorted_first)
        else:
            g = ops.take_along_axis(x, perm, 1)
            outs.append(_canonical_float(g) if i < num_keys else g)
    if return_argsort:
        outs.append(perm)
    return tuple(outs)
