"""take_along_axis (mirror of tallax/_src/gather.py:59-83)."""
from tallax_b200._src import ops


def take_along_axis(values, indices, axis, interpret: bool = False):
    """out[b, j] = values[b, indices[b, j]] (axis=1) or out[i, b] = values[indices[i, b], b] (axis=0).

    2-D only; an index outside the axis yields 0, as in the reference (gather.py:17-35).
    """
    if axis not in (0, 1):
        raise ValueError("axis must be 0 or 1")
    return ops.take_along_axis(values, indices, axis)
