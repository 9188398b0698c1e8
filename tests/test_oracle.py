"""CPU checks of the oracle itself: known-answer vectors and internal consistency."""
import numpy as np
import pytest

from oracle import tallax_oracle as o


def test_threefry_known_answers():
    for key, ctr, exp in o.THREEFRY_KAT:
        r0, r1 = o.threefry2x32(key, np.uint32(ctr[0]), np.uint32(ctr[1]))
        assert (int(r0), int(r1)) == exp


def test_key_transform_orders_like_floats():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1000).astype(np.float32)
    x[:6] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45]
    k = o.sortable_key_u32(x)
    fin = ~np.isnan(x)
    order = np.argsort(k[fin], kind="stable")
    assert np.all(np.diff(x[fin][order]) >= 0)
    assert k[0] == k[1]  # -0 folds onto +0
    assert k[4] == 0xFFFFFFFF and np.all(k[fin] < k[4])  # NaN is the greatest key
    back = o.key_u32_to_f32(k)
    assert np.array_equal(back[fin], np.where(x[fin] == 0, 0.0, x[fin]).astype(np.float32))


def test_sort_matches_numpy_stable_sort():
    keys, payload = o.make_sort_inputs(4, 1000)
    sk, sp = o.sort([keys, payload], 1, is_stable=True)
    idx = np.argsort(keys, axis=1, kind="stable")
    assert np.array_equal(sk, np.take_along_axis(keys, idx, 1))
    assert np.array_equal(sp, idx)
    dk, dp = o.sort([keys, payload], 1, is_stable=True, descending=True)
    assert np.all(np.diff(dk, axis=1) <= 0)
    ties = dk[:, 1:] == dk[:, :-1]
    assert np.all(np.diff(dp, axis=1)[ties] > 0)  # descending keys, ascending index on ties


def test_two_key_sort():
    rng = np.random.default_rng(1)
    a = rng.integers(0, 4, (3, 200)).astype(np.int32)
    b = rng.standard_normal((3, 200)).astype(np.float32)
    sa, sb = o.sort([a, b], 2)
    for r in range(3):
        ref = sorted(zip(a[r].tolist(), b[r].tolist()))
        assert [x for x, _ in ref] == sa[r].tolist()
        assert np.array_equal(np.array([y for _, y in ref], np.float32), sb[r])


def test_topk_ties_lower_index_first():
    x = np.array([[1, 3, 3, 2, 3, 0]], np.float32)
    v, i = o.top_k(x, 4)
    assert v.tolist() == [[3, 3, 3, 2]] and i.tolist() == [[1, 2, 4, 3]]


def test_gather_out_of_range_is_zero():
    v = np.arange(12, dtype=np.float32).reshape(3, 4) + 1
    i = np.array([[0, 3, 4, -1]] * 3, np.int32)
    out = o.take_along_axis(v, i, 1)
    assert out[:, 2].tolist() == [0, 0, 0] and out[:, 3].tolist() == [0, 0, 0] and out[1, 1] == 8


def test_sparse_uniform_equals_dense():
    key = (42, 7)
    dense = o.dense_uniform(key, (16, 256))
    i0 = np.random.default_rng(0).integers(0, 16, (8, 128))
    i1 = np.random.default_rng(1).integers(0, 256, (8, 128))
    sp = o.sparse_random_uniform(key, (i0, i1), 256, minval=o.F32_TINY, maxval=1.0)
    assert np.array_equal(sp, dense[i0, i1])
    assert dense.min() >= o.F32_TINY and dense.max() < 1.0


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_sampler_forms_agree(dtype):
    x, tk, tp, T, noise = o.make_sampling_inputs(B=12, V=4096, seed=5, dtype=dtype)
    T[3] = 1e-6  # a greedy row
    dense = o.sample(x, tk, tp, T, noise=noise)
    assert dense[3] == np.argmax(x[3].astype(np.float32))
    tk128 = np.clip(tk, 1, 128)
    assert np.array_equal(o.sample(x, tk128, tp, T, noise=noise), o.sample_two_stage(x, tk128, tp, T, noise=noise))
    tk50 = np.clip(tk, 1, 50)
    assert np.array_equal(o.sample(x, tk50, tp, T, noise=noise), o.sample_vocab_sharded(x, 4, tk50, tp, T, noise))
    # the key-based noise path equals the dense-tensor path fed with the dense threefry tensor
    key = (123, 456)
    u = o.dense_uniform(key, x.shape)
    assert np.array_equal(o.sample(x, tk, tp, T, rng_key=key), o.sample(x, tk, tp, T, noise=u))


def test_top_p_mask_literal_form():
    x = np.sort(np.random.default_rng(3).standard_normal((16, 5)).astype(np.float32), axis=0)[::-1].copy()
    p = np.array([0.1, 0.5, 0.9, 0.99, 0.3], np.float32)
    m = o.top_p_mask(x, p, -1e12)
    for b in range(5):
        e = np.exp(x[:, b].astype(np.float64) - x[0, b])
        cs = np.cumsum(e / e.sum())
        t = int((cs < p[b]).sum())
        assert np.array_equal(m[:, b] > -1e11, x[:, b] >= x[t, b])
