"""Multi-operand top-k for k <= 128 and arg-max with payloads
(mirror of tallax/_src/bitonic_top_k.py:43-97, 343-402)."""
from __future__ import annotations

from tallax_b200._src import ops
from tallax_b200._src.sort import canonicalize_operand, sort

NUM_LANES = 128


def bitonic_top_k(operand, k: int = NUM_LANES, num_keys: int = 1, descending: bool = True, interpret: bool = False):
    """Top-k of same-shape operands; the first `num_keys` are lexicographic keys and
    every operand is permuted alike.  Ties: lower column first."""
    if k > NUM_LANES:
        raise ValueError(f"bitonic_topk only supports k<=NUM_LANES={NUM_LANES}, got k={k}")
    if not descending:
        raise NotImplementedError
    operands, shape = canonicalize_operand(operand)
    k = min(k, shape[1])
    if num_keys == 1:
        vals, idx = ops.top_k(operands[0], k)
        return (vals,) + tuple(ops.take_along_axis(x, idx, 1) for x in operands[1:])
    outs = sort(operands, num_keys=num_keys, is_stable=True, descending=True, return_argsort=True)
    perm = outs[-1][:, :k].contiguous()
    return tuple(ops.take_along_axis(x, perm, 1) for x in operands)


def max_arrays(operands, num_keys: int, axis: int):
    """Lexicographic arg-max along `axis` carrying every operand; returns 1-D arrays."""
    operands, shape = canonicalize_operand(operands)
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1")
    if num_keys == 1:
        win = ops.argmax(operands[0], axis)
        idx = win.reshape(-1, 1) if axis == 1 else win.reshape(1, -1)
        return [ops.take_along_axis(x, idx, axis).reshape(-1) for x in operands]
    if axis == 0:
        operands = [x.t().contiguous() for x in operands]
    outs = sort(operands, num_keys=num_keys, is_stable=True, descending=True)
    return [o[:, 0].contiguous() for o in outs]
