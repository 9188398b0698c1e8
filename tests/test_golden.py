"""The oracle and the CUDA library against fixtures produced by the REFERENCE's own value-level code.

tests/golden/reference_value_level.npz holds outputs of the reference's `*_arrays` functions (the
bodies of its Pallas kernels), run from the reference checkout with jax.numpy mapped onto NumPy
(tests/golden/make_golden.py).  The CPU tests pin the oracle to them; the GPU tests compare
the CUDA library with the same stored outputs.
"""
import os

import numpy as np
import pytest

from oracle import tallax_oracle as o

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_value_level.npz"))
RTOL_CUMSUM, ATOL_CUMSUM = 1e-3, 1e-6   # the reference's own cumsum tolerance (tests/cumsum_test.py:31)


def _near_threshold_columns(x, p):
    e = np.exp(x.astype(np.float64) - x[:1].astype(np.float64))
    cs = np.cumsum(e / e.sum(0), axis=0)
    return np.abs(cs - p[None, :].astype(np.float64)).min(axis=0) < 1e-5   # f32 cumulative sums in the reference


# ------------------------------------------------------------------------------------------ CPU: oracle
def test_key_transform_orders_like_the_reference():
    x, ref = G["key_in"], G["key_sortable_int"].astype(np.int64)
    mine = o.sortable_key_u32(x).astype(np.int64)
    # same order and same equivalence classes (the reference uses signed keys, the oracle unsigned ones)
    assert np.array_equal(np.argsort(ref, kind="stable"), np.argsort(mine, kind="stable"))
    assert np.array_equal(ref[:, None] == ref[None, :], mine[:, None] == mine[None, :])
    back = o.key_u32_to_f32(o.sortable_key_u32(x))
    assert np.array_equal(back, G["key_roundtrip"], equal_nan=True)


def test_cumsum_matches_reference():
    for i in range(5):
        axis, rev = (int(v) for v in G[f"cumsum{i}_meta"])
        assert np.array_equal(o.cumsum(G[f"cumsum{i}_i32_in"], axis, bool(rev)), G[f"cumsum{i}_i32_out"])
        np.testing.assert_allclose(o.cumsum(G[f"cumsum{i}_f32_in"], axis, bool(rev)), G[f"cumsum{i}_f32_out"],
                                   rtol=RTOL_CUMSUM, atol=1e-4)


def test_gather_matches_reference_including_out_of_range():
    for i in range(3):
        got = o.take_along_axis(G[f"gather{i}_val"], G[f"gather{i}_idx"], int(G[f"gather{i}_axis"]))
        assert np.array_equal(got, G[f"gather{i}_out"])


def test_max_arrays_matches_reference():
    for i in range(4):
        v, axis = G[f"max{i}_val"], int(G[f"max{i}_axis"])
        iota = np.broadcast_to(np.arange(v.shape[axis], dtype=np.int32).reshape((-1, 1) if axis == 0 else (1, -1)),
                               v.shape)
        got = o.max_arrays([v, iota], 1, axis)
        assert np.array_equal(got[0], G[f"max{i}_out_val"]) and np.array_equal(got[1], G[f"max{i}_out_idx"])


def test_sparse_uniform_matches_reference():
    for i in range(3):
        lo, hi = (float(v) for v in G[f"uniform{i}_range"])
        key = tuple(int(v) for v in G[f"uniform{i}_key"].reshape(-1))
        got = o.sparse_random_uniform(key, (G[f"uniform{i}_i0"], G[f"uniform{i}_i1"]), 256, lo, hi)
        assert np.array_equal(got, G[f"uniform{i}_out"])


def test_top_p_mask_matches_reference():
    x, p = G["topp_in"], G["topp_p"]
    got = o.top_p_mask(x, p, -1e12)
    ok = ~_near_threshold_columns(x, p)
    assert ok.sum() >= 28 and np.array_equal(got[:, ok], G["topp_out"][:, ok])


def test_top_p_and_sample_matches_reference():
    V, off = (int(v) for v in G["sample_meta"])
    key = tuple(int(v) for v in G["sample_key"].reshape(-1))
    got, flags = o.top_p_and_sample(G["sample_vals"], G["sample_idx"], G["sample_top_p"], G["sample_temp"],
                                    vocab_size=V, replace_val=-1e12, rng_key=key, dim0_offset=off, return_flags=True)
    # the reference sums f32 probabilities and takes f32 logs: rows within 1e-5 of the threshold may differ
    bad = (got != G["sample_tokens"]) & ~flags
    assert bad.sum() <= 1, (np.flatnonzero(bad), got[bad], G["sample_tokens"][bad])


def test_sparse_categorical_matches_reference():
    lg, rws, cols = G["cat_logits"], G["cat_rows"], G["cat_cols"]
    u = o.sparse_random_uniform((5, 6), (rws, cols), 256, minval=o.F32_TINY, maxval=1.0)
    win = np.argmax(lg + o.gumbel_from_uniform(u), axis=1)
    assert np.array_equal(np.take_along_axis(cols, win[:, None], 1)[:, 0], G["cat_out1"])
    assert np.array_equal(np.take_along_axis(rws, win[:, None], 1)[:, 0], G["cat_out0"])


# ------------------------------------------------------------------------------------------ GPU: library
@pytest.mark.gpu
def test_gpu_simple_ops_match_reference(cuda):
    from tallax_b200 import tax, tumpy
    from tallax_b200._src.bitonic_top_k import max_arrays
    from tallax_b200._src.sparse_random import sparse_random_categorical, sparse_random_uniform
    from tests.conftest import to_dev, to_np

    for i in range(5):
        axis, rev = (int(v) for v in G[f"cumsum{i}_meta"])
        assert np.array_equal(to_np(tax.cumsum(to_dev(G[f"cumsum{i}_i32_in"], cuda), axis, bool(rev))),
                              G[f"cumsum{i}_i32_out"])
        np.testing.assert_allclose(to_np(tax.cumsum(to_dev(G[f"cumsum{i}_f32_in"], cuda), axis, bool(rev))),
                                   G[f"cumsum{i}_f32_out"], rtol=RTOL_CUMSUM, atol=1e-4)
    for i in range(3):
        got = tumpy.take_along_axis(to_dev(G[f"gather{i}_val"], cuda), to_dev(G[f"gather{i}_idx"], cuda),
                                    int(G[f"gather{i}_axis"]))
        assert np.array_equal(to_np(got), G[f"gather{i}_out"])
    for i in range(4):
        v, axis = G[f"max{i}_val"], int(G[f"max{i}_axis"])
        iota = np.broadcast_to(np.arange(v.shape[axis], dtype=np.int32).reshape((-1, 1) if axis == 0 else (1, -1)),
                               v.shape).copy()
        got = max_arrays([to_dev(v, cuda), to_dev(iota, cuda)], num_keys=1, axis=axis)
        assert np.array_equal(to_np(got[0]), G[f"max{i}_out_val"]) and np.array_equal(to_np(got[1]), G[f"max{i}_out_idx"])
    for i in range(3):
        lo, hi = (float(v) for v in G[f"uniform{i}_range"])
        key = tuple(int(v) for v in G[f"uniform{i}_key"].reshape(-1))
        got = sparse_random_uniform(key, [to_dev(G[f"uniform{i}_i0"], cuda), to_dev(G[f"uniform{i}_i1"], cuda)], 256,
                                    minval=lo, maxval=hi)
        assert np.array_equal(to_np(got), G[f"uniform{i}_out"])
    got = sparse_random_categorical((5, 6), to_dev(G["cat_logits"], cuda),
                                    [to_dev(G["cat_rows"], cuda), to_dev(G["cat_cols"], cuda)], 256, axis=1)
    assert np.array_equal(to_np(got[1]), G["cat_out1"]) and np.array_equal(to_np(got[0]), G["cat_out0"])


@pytest.mark.gpu
def test_gpu_sampler_matches_reference(cuda):
    from tallax_b200 import sampling
    from tests.conftest import to_dev, to_np

    x, p = G["topp_in"], G["topp_p"]
    got = to_np(sampling.top_p_mask(topk_logits=to_dev(x, cuda), p=to_dev(p, cuda), replace_val=-1e12, axis=0))
    ok = ~_near_threshold_columns(x, p)
    assert np.array_equal(got[:, ok], G["topp_out"][:, ok])

    V, off = (int(v) for v in G["sample_meta"])
    key = tuple(int(v) for v in G["sample_key"].reshape(-1))
    tok = sampling.top_p_and_sample(to_dev(G["sample_vals"], cuda), to_dev(G["sample_idx"], cuda), key,
                                    to_dev(G["sample_top_p"], cuda), to_dev(G["sample_temp"], cuda), vocab_size=V,
                                    replace_val=-1e12, dim0_offset=off)
    _, flags = o.top_p_and_sample(G["sample_vals"], G["sample_idx"], G["sample_top_p"], G["sample_temp"],
                                  vocab_size=V, replace_val=-1e12, rng_key=key, dim0_offset=off, return_flags=True)
    bad = (to_np(tok) != G["sample_tokens"]) & ~flags
    assert bad.sum() <= 1
