"""GPU parity: gather, cumsum, arg-max, indexed noise against the oracle (bit-exact unless stated)."""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200 import tax, tumpy
from tallax_b200._src.bitonic_top_k import max_arrays
from tallax_b200._src.sparse_random import sparse_random_categorical, sparse_random_uniform
from tests.conftest import exact_match, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("num_tokens", [8, 16, 13])
@pytest.mark.parametrize("vocab_size", [128, 256, 300])
@pytest.mark.parametrize("k", [64, 128, 200, 300])
@pytest.mark.parametrize("axis", [0, 1])
def test_take_along_axis(cuda, num_tokens, vocab_size, k, axis):
    rng = np.random.default_rng(0)
    if axis == 1:
        values = rng.standard_normal((num_tokens, vocab_size)).astype(np.float32)
        indices = rng.integers(0, vocab_size, (num_tokens, k)).astype(np.int32)
    else:
        values = rng.standard_normal((vocab_size, num_tokens)).astype(np.float32)
        indices = rng.integers(0, vocab_size, (k, num_tokens)).astype(np.int32)
    out = tumpy.take_along_axis(to_dev(values, cuda), to_dev(indices, cuda), axis)
    assert np.array_equal(to_np(out), o.take_along_axis(values, indices, axis))


@pytest.mark.parametrize("dtype", ["f32", "bf16", "i32"])
def test_take_along_axis_large_and_out_of_range(cuda, dtype):
    rng = np.random.default_rng(1)
    values = rng.standard_normal((8, 2048)).astype(np.float32) * 100
    values = {"f32": values, "bf16": values.astype(o.bfloat16), "i32": values.astype(np.int32)}[dtype]
    indices = rng.integers(-50, 2100, (8, 1027)).astype(np.int32)  # some negative, some too large, ragged width
    out = tumpy.take_along_axis(to_dev(values, cuda), to_dev(indices, cuda), 1)
    assert exact_match(to_np(out), o.take_along_axis(values, indices, 1))


def test_take_along_axis_empty_and_errors(cuda):
    v = torch.zeros((4, 16), device=cuda)
    assert tumpy.take_along_axis(v, torch.zeros((4, 0), dtype=torch.int32, device=cuda), 1).shape == (4, 0)
    with pytest.raises(ValueError):
        tumpy.take_along_axis(v, torch.zeros((5, 3), dtype=torch.int32, device=cuda), 1)


def test_take_along_axis_wide_rows(cuda):
    # the shape class of the benchmark configuration: long value rows, a few thousand indices per row
    rng = np.random.default_rng(3)
    values = rng.standard_normal((16, 262144)).astype(np.float32)
    indices = rng.integers(0, 262144, (16, 4096)).astype(np.int32)
    out = tumpy.take_along_axis(to_dev(values, cuda), to_dev(indices, cuda), 1)
    assert np.array_equal(to_np(out), np.take_along_axis(values, indices.astype(np.int64), 1))


@pytest.mark.parametrize("shape", [(8, 128), (16, 256), (128, 8), (256, 16), (13, 167), (3, 100001)])
@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("dtype", ["f32", "i32"])
@pytest.mark.parametrize("reverse", [False, True])
def test_cumsum(cuda, shape, axis, dtype, reverse):
    rng = np.random.default_rng(42)
    if dtype == "f32":
        x = rng.standard_normal(shape).astype(np.float32)
    else:
        x = rng.integers(0, 100, shape).astype(np.int32)
    out = to_np(tax.cumsum(to_dev(x, cuda), axis=axis, reverse=reverse))
    if dtype == "i32":
        assert np.array_equal(out, o.cumsum(x, axis, reverse))
    elif max(shape) <= 256:
        # the reference's own shapes and its own tolerance against lax.cumsum (tests/cumsum_test.py:31)
        np.testing.assert_allclose(out, o.cumsum(x, axis, reverse), rtol=1e-3, atol=1e-6)
    else:
        # long rows: f32 rounding grows with the length for any summation order, so compare with an
        # f64 accumulation at a tolerance of a few f32 ulps of the largest partial sum
        ref = o.cumsum(x, axis, reverse, accum=np.float64)
        assert np.abs(out - ref).max() <= 64 * np.finfo(np.float32).eps * np.abs(ref).max()


@pytest.mark.parametrize("shape", [(8, 128), (16, 256), (128, 8), (256, 16), (256, 256), (173, 195)])
@pytest.mark.parametrize("dtype", ["f32", "i32"])
@pytest.mark.parametrize("axis", [0, 1])
def test_max_arrays(cuda, shape, dtype, axis):
    rng = np.random.default_rng(1 + axis)
    arr = rng.standard_normal(shape).astype(np.float32) if dtype == "f32" else rng.integers(0, 1000, shape).astype(
        np.int32)
    idx = np.broadcast_to(np.arange(shape[axis]).reshape((-1, 1) if axis == 0 else (1, -1)), shape).astype(np.int32)
    got = max_arrays([to_dev(arr, cuda), to_dev(idx.copy(), cuda)], num_keys=1, axis=axis)
    exp = o.max_arrays([arr, idx], 1, axis)
    assert np.array_equal(to_np(got[0]), exp[0]) and np.array_equal(to_np(got[1]), exp[1])


def test_max_arrays_two_keys(cuda):
    rng = np.random.default_rng(5)
    a = rng.integers(0, 3, (16, 64)).astype(np.int32)
    b = rng.standard_normal((16, 64)).astype(np.float32)
    c = np.broadcast_to(np.arange(64, dtype=np.int32), (16, 64)).copy()
    got = max_arrays([to_dev(a, cuda), to_dev(b, cuda), to_dev(c, cuda)], num_keys=2, axis=1)
    exp = o.max_arrays([a, b, c], 2, 1)
    for g, e in zip(got, exp):
        assert np.array_equal(to_np(g), e)


@pytest.mark.parametrize("seed", [42, 123, 456])
@pytest.mark.parametrize("minval,maxval", [(0.0, 1.0), (-1.0, 1.0), (5.0, 10.0)])
def test_sparse_random_uniform(cuda, seed, minval, maxval):
    rng = np.random.default_rng(seed)
    key = (seed, seed * 7 + 1)
    i0 = rng.integers(0, 16, (8, 128)).astype(np.int32)
    i1 = rng.integers(0, 256, (8, 128)).astype(np.int32)
    got = to_np(sparse_random_uniform(key, [to_dev(i0, cuda), to_dev(i1, cuda)], 256, minval=minval, maxval=maxval))
    assert np.array_equal(got, o.sparse_random_uniform(key, (i0, i1), 256, minval, maxval))


def test_sparse_random_uniform_counter_wraps_like_uint32(cuda):
    i0 = np.array([[40000, 65535]], np.int32)
    i1 = np.array([[7, 123456]], np.int32)
    got = to_np(sparse_random_uniform((1, 2), [to_dev(i0, cuda), to_dev(i1, cuda)], 200000))
    assert np.array_equal(got, o.sparse_random_uniform((1, 2), (i0, i1), 200000))


@pytest.mark.parametrize("seed", [789, 321, 654])
@pytest.mark.parametrize("axis", [0, 1])
def test_sparse_random_categorical(cuda, seed, axis):
    rng = np.random.default_rng(seed)
    key = (seed, 99)
    batch, dense, sparse = 16, 256, 128
    logits = rng.standard_normal((batch, sparse)).astype(np.float32)
    choices = np.stack([rng.choice(dense, sparse, replace=False) for _ in range(batch)]).astype(np.int32)
    rows = np.broadcast_to(np.arange(batch, dtype=np.int32)[:, None], (batch, sparse)).copy()
    if axis == 1:
        lg, i0, i1, dim1 = logits, rows, choices, dense
    else:
        lg, i0, i1, dim1 = logits.T.copy(), choices.T.copy(), rows.T.copy(), batch
    got = sparse_random_categorical(key, to_dev(lg, cuda), [to_dev(i0, cuda), to_dev(i1, cuda)], dim1, axis=axis)
    u = o.sparse_random_uniform(key, (i0, i1), dim1, minval=o.F32_TINY, maxval=1.0)
    y = lg + o.gumbel_from_uniform(u)
    win = np.argmax(y, axis=axis)
    sel = win[:, None] if axis == 1 else win[None, :]
    assert np.array_equal(to_np(got[0]), np.take_along_axis(i0, sel, axis).reshape(-1))
    assert np.array_equal(to_np(got[1]), np.take_along_axis(i1, sel, axis).reshape(-1))
