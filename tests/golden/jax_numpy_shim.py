"""A NumPy stand-in for the small part of the jax API that the reference's VALUE-LEVEL functions use.

JAX cannot be installed here, but the reference's `*_arrays` functions (the bodies of its
Pallas kernels) are ordinary array code: with `jax.numpy` mapped onto NumPy they run as
written.  `install()` puts fake `jax` modules into sys.modules so that the reference tree can
be imported; `make_golden.py` then runs the reference's own code on seeded inputs and stores
the results as fixtures.  Only used to GENERATE fixtures: the tests read the stored files.

What is faked faithfully: dtypes, where/pad/concatenate/split/take_along_axis/exp/log/...,
lax.broadcasted_iota / slice_in_dim / shift_right_logical / bitcast_convert_type, jax.tree.
What is NOT jax: `threefry2x32_p.bind` is the restatement in oracle/tallax_oracle.py (pinned by
the Random123 known-answer vectors), and every Pallas entry point raises.
"""
from __future__ import annotations

import sys
import types

import ml_dtypes
import numpy as np


def _tree_leaves(t):
    if isinstance(t, (list, tuple)):
        out = []
        for x in t:
            out.extend(_tree_leaves(x))
        return out
    return [t]


def _tree_map(f, *trees):
    t0 = trees[0]
    if isinstance(t0, (list, tuple)):
        return type(t0)(_tree_map(f, *[t[i] for t in trees]) for i in range(len(t0)))
    return f(*trees)


class _Structure:
    def __init__(self, n):
        self.n = n


def _tree_structure(t):
    return _Structure(len(t))


def _tree_transpose(outer, inner, tree):
    # list of lists [outer][inner] -> [inner][outer]
    return [[tree[o][i] for o in range(outer.n)] for i in range(inner.n)]


def _not_available(*a, **k):
    raise RuntimeError("Pallas / XLA entry points are not available in the NumPy stand-in")


class _Passthrough:
    """Decorator factories such as jax.jit / functools.partial(jit, ...) become identity."""

    def __call__(self, fn=None, **kwargs):
        if fn is None:
            return lambda f: f
        return fn


class JArr(np.ndarray):
    """ndarray with jax's value semantics: `a += b` rebinds `a` to a new array instead of
    writing through (the reference relies on that: it updates slices obtained from jnp.split)."""

    def __iadd__(self, other): return self + other
    def __isub__(self, other): return self - other
    def __imul__(self, other): return self * other
    def __iand__(self, other): return self & other
    def __ior__(self, other): return self | other
    def __ixor__(self, other): return self ^ other
    def __itruediv__(self, other): return self / other


def as_jax(x):
    return np.asarray(x).view(JArr)


def _demote(x):
    """jax works in 32 bits by default: results that NumPy made 64-bit wide go back to 32;
    arrays come back with jax's value semantics."""
    if isinstance(x, np.ndarray):
        if x.dtype == np.int64:
            x = x.astype(np.int32)
        elif x.dtype == np.float64:
            x = x.astype(np.float32)
        elif x.dtype == np.uint64:
            x = x.astype(np.uint32)
        return x.view(JArr)
    if isinstance(x, np.generic):
        if x.dtype == np.int64:
            return np.int32(x)
        if x.dtype == np.float64:
            return np.float32(x)
        return x
    if isinstance(x, (list, tuple)):
        return type(x)(_demote(v) for v in x)
    return x


def _wrap32(fn):
    def inner(*a, **k):
        return _demote(fn(*a, **k))
    return inner


def install():
    from oracle import tallax_oracle as o

    jnp = types.ModuleType("jax.numpy")
    for name in ("where isnan zeros ones zeros_like ones_like pad concatenate split take_along_axis exp log arange "
                 "broadcast_to array reshape bitwise_xor bitwise_and bitwise_or maximum minimum sum cumsum sort "
                 "argsort unique array_equal stack full asarray abs sqrt transpose expand_dims squeeze").split():
        setattr(jnp, name, _wrap32(getattr(np, name)))
    jnp.float32, jnp.int32, jnp.uint32, jnp.uint16, jnp.int16 = np.float32, np.int32, np.uint32, np.uint16, np.int16
    jnp.bool_, jnp.floating, jnp.integer, jnp.ndarray = np.bool_, np.floating, np.integer, np.ndarray
    jnp.bfloat16 = ml_dtypes.bfloat16
    jnp.nan, jnp.inf = np.nan, np.inf
    jnp.iinfo = np.iinfo
    jnp.finfo = lambda dt: ml_dtypes.finfo(dt)
    jnp.issubdtype = lambda a, b: (np.issubdtype(a, b) if a != ml_dtypes.bfloat16 else b in (np.floating, np.inexact))

    lax = types.ModuleType("jax.lax")

    def broadcasted_iota(dtype, shape, dim):
        idx = np.arange(shape[dim], dtype=dtype)
        view = [1] * len(shape)
        view[dim] = shape[dim]
        return np.broadcast_to(idx.reshape(view), shape).copy().view(JArr)

    def slice_in_dim(x, start, limit, axis=0):
        sl = [slice(None)] * x.ndim
        sl[axis] = slice(start, limit)
        return np.asarray(x)[tuple(sl)].view(JArr)

    lax.broadcasted_iota = broadcasted_iota
    lax.slice_in_dim = slice_in_dim
    lax.shift_right_logical = lambda x, s: (np.asarray(x, np.uint32) >> np.uint32(s)).astype(np.uint32).view(JArr)
    lax.bitwise_or = np.bitwise_or
    lax.bitcast_convert_type = lambda x, dt: np.asarray(x).view(dt).view(JArr)
    lax.convert_element_type = lambda x, dt: np.asarray(x).astype(dt)[()]
    lax.max = np.maximum
    lax.cumsum = lambda x, axis=0, reverse=False: o.cumsum(x, axis, reverse)
    lax.fori_loop = lambda lo, hi, body, init: __import__("functools").reduce(lambda c, i: body(i, c), range(lo, hi), init)
    lax.sort = _not_available

    jax = types.ModuleType("jax")
    jax.numpy, jax.lax = jnp, lax
    jax.Array = np.ndarray
    jax.jit = _Passthrough()
    jit = jax.jit
    jax.default_backend = lambda: "cpu"
    jax.ShapeDtypeStruct = lambda shape, dtype: (shape, dtype)
    tree = types.ModuleType("jax.tree")
    tree.map, tree.leaves, tree.structure, tree.transpose = _tree_map, _tree_leaves, _tree_structure, _tree_transpose
    jax.tree = tree
    rnd = types.ModuleType("jax.random")
    rnd.key_data = lambda k: np.asarray(k, np.uint32)
    jax.random = rnd

    pallas = types.ModuleType("jax.experimental.pallas")
    pallas.cdiv = lambda a, b: -(-a // b)
    pallas.dslice = lambda start, size: slice(int(start), int(start) + int(size))   # a dynamic slice of an array
    pallas.pallas_call = _not_available
    pallas.BlockSpec = lambda *a, **k: None
    pallas.when = _not_available
    pallas.loop = _not_available
    tpu = types.ModuleType("jax.experimental.pallas.tpu")
    for n in ("VMEM", "SMEM", "ANY", "CompilerParams", "async_copy", "SemaphoreType"):
        setattr(tpu, n, _not_available)
    pallas.tpu = tpu
    experimental = types.ModuleType("jax.experimental")
    experimental.pallas = pallas
    cp = types.ModuleType("jax.experimental.custom_partitioning")
    cp.custom_partitioning = lambda f: f
    sharding = types.ModuleType("jax.sharding")
    sharding.Mesh = sharding.NamedSharding = sharding.PartitionSpec = object
    extend = types.ModuleType("jax.extend")
    ext_random = types.ModuleType("jax.extend.random")

    class _Threefry:
        @staticmethod
        def bind(k1, k2, hi, lo):
            key = (int(np.asarray(k1).reshape(-1)[0]), int(np.asarray(k2).reshape(-1)[0]))
            return o.threefry2x32(key, hi, lo)

    ext_random.threefry2x32_p = _Threefry
    extend.random = ext_random
    jax.experimental, jax.extend, jax.sharding = experimental, extend, sharding

    mods = {
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.tree": tree, "jax.random": rnd,
        "jax.experimental": experimental, "jax.experimental.pallas": pallas, "jax.experimental.pallas.tpu": tpu,
        "jax.experimental.custom_partitioning": cp, "jax.sharding": sharding, "jax.extend": extend,
        "jax.extend.random": ext_random,
    }
    sys.modules.update(mods)
    return jax
