"""numpy-like wrappers (mirror of tallax/tumpy.py:6-112): sort, argsort, take_along_axis."""
from tallax_b200._src.sort import sort as _lax_sort
from tallax_b200._src.gather import take_along_axis as _take_along_axis


def _prepare(a, axis):
    if axis is None:
        work = a.reshape(-1)
        return work, work.shape, work.numel()
    canonical = axis if axis >= 0 else axis + a.ndim
    if canonical != a.ndim - 1:
        raise ValueError("tumpy only supports sorting along the last axis.")
    return a, a.shape, a.shape[-1]


def sort(a, axis=-1, kind=None, order=None, stable=True, descending=False, interpret=False):
    """Sort along the last axis (tumpy.py:6-52); `kind`, `order`, `interpret` are accepted and ignored."""
    work, target_shape, n = _prepare(a, axis)
    (out,) = _lax_sort(work.reshape(-1, n), num_keys=1, is_stable=stable, descending=descending,
                       return_argsort=False)
    return out.reshape(target_shape)


def argsort(a, axis=-1, kind=None, order=None, stable=True, descending=False, interpret=False):
    """Indices that sort along the last axis (tumpy.py:54-97)."""
    work, target_shape, n = _prepare(a, axis)
    _, idx = _lax_sort(work.reshape(-1, n), num_keys=1, is_stable=stable, descending=descending,
                       return_argsort=True)
    return idx.reshape(target_shape)


def take_along_axis(arr, indices, axis, interpret=False):
    """tumpy.py:99-112."""
    return _take_along_axis(arr, indices, axis)
