"""cumsum (mirror of tallax/_src/cumsum.py:75-101)."""
from tallax_b200._src import ops


def cumsum(arr, axis, reverse: bool = False, interpret: bool = False):
    """Inclusive prefix sum of a 2-D array along `axis`, optionally reversed."""
    if axis < 0:
        axis += arr.ndim
    return ops.cumsum(arr, axis, reverse)
