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
                                   rtol=RTOL_CUMSUM, atol=ATOL_CUMSUM)


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
    # (the reference sums f32 probabilities and takes f32 logs; no row of this fixture comes close enough to
    # its threshold, or to a tie of two scores, for that to show)
    bad = (got != G["sample_tokens"]) & ~flags
    assert bad.sum() == 0, (np.flatnonzero(bad), got[bad], G["sample_tokens"][bad])


def test_sparse_categorical_matches_reference():
    lg, rws, cols = G["cat_logits"], G["cat_rows"], G["cat_cols"]
    u = o.sparse_random_uniform((5, 6), (rws, cols), 256, minval=o.F32_TINY, maxval=1.0)
    win = np.argmax(lg + o.gumbel_from_uniform(u), axis=1)
    assert np.array_equal(np.take_along_axis(cols, win[:, None], 1)[:, 0], G["cat_out1"])
    assert np.array_equal(np.take_along_axis(rws, win[:, None], 1)[:, 0], G["cat_out0"])


def _pairs(name):
    return (G[f"cas_{name}_lk"], G[f"cas_{name}_rk"], G[f"cas_{name}_lp"], G[f"cas_{name}_rp"])


def _oracle_pairs(num_keys, descending):
    """Every (left, right) column pair of the compare_and_swap fixture as a row of two, sorted by the oracle."""
    k2 = np.stack([G["cas_kl"].reshape(-1), G["cas_kr"].reshape(-1)], axis=1)
    p2 = np.stack([G["cas_pl"].reshape(-1), G["cas_pr"].reshape(-1)], axis=1)
    ks, ps = o.sort([k2, p2], num_keys=num_keys, descending=descending)
    shape = G["cas_kl"].shape
    return ks[:, 0].reshape(shape), ks[:, 1].reshape(shape), ps[:, 0].reshape(shape), ps[:, 1].reshape(shape)


def test_sort_comparator_matches_reference_compare_and_swap():
    """sort.py:39-102: the oracle's order of two elements is the reference comparator's, for one and two keys,
    static and per-element directions.  With the payload as second key no pair is a full tie; with one key the
    pairs whose keys tie are left out (the reference's network order there is not the stable one)."""
    tie = G["cas_kl"] == G["cas_kr"]
    assert tie.sum() > 50 and (~tie).sum() > 500
    for name, nk, desc in (("asc1", 1, False), ("desc1", 1, True), ("asc2", 2, False), ("desc2", 2, True)):
        ref = _pairs(name)
        mine = _oracle_pairs(nk, desc)
        sel = ~tie if nk == 1 else np.ones_like(tie)
        for r, m in zip(ref, mine):
            assert np.array_equal(r[sel], m[sel]), name
    dyn = G["cas_dyn"].astype(bool)
    for name, nk in (("dyn1", 1), ("dyn2", 2)):
        ref = _pairs(name)
        up, down = _oracle_pairs(nk, False), _oracle_pairs(nk, True)
        sel = ~tie if nk == 1 else np.ones_like(tie)
        for r, a, d in zip(ref, up, down):
            assert np.array_equal(r[sel], np.where(dyn, d, a)[sel]), name


def test_sort_matches_a_bitonic_network_of_reference_comparators():
    """A 64-wide bitonic network whose every exchange is the reference's compare_and_swap on (value, column):
    the oracle's sort gives the same rows, and for the ascending one its stable single-key sort gives the same
    permutation (ties -> lower column first)."""
    v = G["net_in"]
    col = np.broadcast_to(np.arange(v.shape[1], dtype=np.int32), v.shape)
    for name, desc in (("asc", False), ("desc", True)):
        val, perm = o.sort([v, col], num_keys=2, descending=desc)
        assert np.array_equal(val, G[f"net_{name}_val"]) and np.array_equal(perm, G[f"net_{name}_col"])
    val, perm = o.sort([v], num_keys=1, is_stable=True, return_argsort=True)
    assert np.array_equal(perm, G["net_asc_col"])


def _bins_as_rows(x, nb):
    """Bin j of a row holds the elements j, j + nb, j + 2 nb, ...: one short row per (row, bin), padded with -inf."""
    rows, n = x.shape
    depth = -(-n // nb)
    pad = np.full((rows, depth * nb), -np.inf, np.float32)
    pad[:, :n] = x
    return pad.reshape(rows, depth, nb).transpose(0, 2, 1).reshape(rows * nb, depth)


def _check_binned(x, nb, vals, glob):
    """vals, glob: [k, rows, nb] top-k values and global indices of every (row, bin), to be compared with the
    reference's binned_top_k.  Values must be equal.  Indices must be equal wherever a value is unique inside
    its bin; among equal values the reference's order is the order in which its sinking sort happened to
    displace them (an element pushed down by a later, larger one lands BELOW an equal element that arrived
    after it), not an index order, so there only the sets can be compared, and at the k-th value only
    membership."""
    ref_v, ref_i = G["binned_vals"], G["binned_idxs"]
    assert np.array_equal(vals, ref_v)
    k, rows, _ = ref_v.shape
    assert np.array_equal(x[np.arange(rows)[None, :, None], glob], vals)       # indices point at their values
    assert np.array_equal(x[np.arange(rows)[None, :, None], ref_i], ref_v)
    assert (glob % nb == np.arange(nb)).all() and (ref_i % nb == np.arange(nb)).all()   # and stay in their bin
    uniq = np.ones_like(ref_v, dtype=bool)
    for a in range(k):
        for b in range(k):
            if a != b:
                uniq[a] &= ref_v[a] != ref_v[b]
    kth_tied = ref_v == ref_v[-1:]                     # the k-th value may tie with elements left out
    assert np.array_equal(glob[uniq & ~kth_tied], ref_i[uniq & ~kth_tied]) and (uniq & ~kth_tied).mean() > 0.5
    inner = ~kth_tied                                  # tie groups entirely inside the top-k: same index sets
    assert np.array_equal(np.sort(np.where(inner, glob, -1), axis=0), np.sort(np.where(inner, ref_i, -1), axis=0))
    # the lower-index-first rule of the oracle differs from the reference's order on some of these bins
    return int((glob != ref_i).sum())


def test_top_k_against_reference_binned_top_k():
    """top_k.py:13-106 on rows with many ties, a ragged last slice included."""
    x, nb = G["binned_in"], 128
    k = G["binned_vals"].shape[0]
    sub = _bins_as_rows(x, nb)
    vals, idx = o.top_k(sub, k)
    j = np.tile(np.arange(nb), x.shape[0])[:, None]
    glob = (j + nb * idx).reshape(x.shape[0], nb, k).transpose(2, 0, 1)
    differing = _check_binned(x, nb, vals.reshape(x.shape[0], nb, k).transpose(2, 0, 1), glob)
    assert differing > 0   # the fixture does exercise tie order: "ties -> lower index" is the oracle's definition,
    #                        one valid answer (the same one jax.lax.top_k gives), not the reference's bin order


def test_bf16_packed_order_matches_reference_pack():
    """utils.py:205-227: ascending order of the reference's packed (bf16 value, index) words is the oracle's
    stable ascending order of the values; unpacking gives the canonical values and the indices back."""
    import ml_dtypes
    x = G["pack_in"].astype(ml_dtypes.bfloat16)
    ref_order = np.argsort(G["pack_packed"].astype(np.int64), axis=1, kind="stable")
    assert np.array_equal(ref_order, o.argsort(x))
    assert np.array_equal(G["pack_unpacked_idx"], np.broadcast_to(np.arange(x.shape[1]), x.shape))
    assert np.array_equal(G["pack_unpacked_val"], o._canon(x).astype(np.float32))
    assert not np.signbit(G["pack_unpacked_val"][0, 1])   # -0 comes back as +0


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
                                   G[f"cumsum{i}_f32_out"], rtol=RTOL_CUMSUM, atol=ATOL_CUMSUM)
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
    assert bad.sum() == 0


@pytest.mark.gpu
def test_gpu_sort_and_top_k_match_reference_comparator_fixtures(cuda):
    import ml_dtypes
    from tallax_b200 import tax
    from tests.conftest import to_dev, to_np

    v = G["net_in"]
    col = np.broadcast_to(np.arange(v.shape[1], dtype=np.int32), v.shape).copy()
    for name, desc in (("asc", False), ("desc", True)):
        val, perm = tax.sort([to_dev(v, cuda), to_dev(col, cuda)], num_keys=2, descending=desc)
        assert np.array_equal(to_np(val), G[f"net_{name}_val"]) and np.array_equal(to_np(perm), G[f"net_{name}_col"])
    out = tax.sort([to_dev(v, cuda)], num_keys=1, is_stable=True, return_argsort=True)
    assert np.array_equal(to_np(out[-1]), G["net_asc_col"])
    # the reference's binned_top_k on rows with many ties
    x, nb = G["binned_in"], 128
    k = G["binned_vals"].shape[0]
    sub = _bins_as_rows(x, nb)
    vals, idx = tax.top_k(to_dev(sub, cuda), k)
    j = np.tile(np.arange(nb), x.shape[0])[:, None]
    glob = (j + nb * to_np(idx)).reshape(x.shape[0], nb, k).transpose(2, 0, 1)
    _check_binned(x, nb, to_np(vals).reshape(x.shape[0], nb, k).transpose(2, 0, 1), glob)
    ov, oi = o.top_k(sub, k)
    assert np.array_equal(to_np(idx), oi)   # and the library's own tie order is the oracle's
    # bf16 keys: the library's stable ascending permutation is the order of the reference's packed words
    xb = G["pack_in"].astype(ml_dtypes.bfloat16)
    out = tax.sort([to_dev(xb, cuda)], num_keys=1, is_stable=True, return_argsort=True)
    assert np.array_equal(to_np(out[-1]), np.argsort(G["pack_packed"].astype(np.int64), axis=1, kind="stable"))
