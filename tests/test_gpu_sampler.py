"""GPU parity: fused sampler, candidate-level sampler, top-p mask, vocab-sharded pipeline.

Token ids must equal the oracle's bit for bit given the same noise, except rows the
oracle flags because their cumulative top-p mass lies within 1e-6 of the threshold.
"""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200 import sampling
from tallax_b200._src import ops
from tests.conftest import to_dev, to_np

pytestmark = pytest.mark.gpu

TOL_NEAR_THRESHOLD = 1e-6  # == oracle.NEAR_THRESHOLD


def _run(cuda, x, tk, tp, T, noise=None, key=None, dim0_offset=0):
    md = sampling.SamplingMetadata(top_k=to_dev(tk, cuda), top_p=to_dev(tp, cuda), temperature=to_dev(T, cuda))
    tok, status = ops.sample(to_dev(x, cuda), md.top_k, md.top_p, md.temperature, rng_key=key,
                             noise=None if noise is None else to_dev(noise, cuda), dim0_offset=dim0_offset,
                             return_status=True)
    return to_np(tok), to_np(status)


def _assert_tokens(got, exp, flags, min_checked=0.9):
    bad = (got != exp) & ~flags
    assert not bad.any(), f"rows {np.flatnonzero(bad)[:10]}: got {got[bad][:10]} expected {exp[bad][:10]}"
    assert (~flags).mean() >= min_checked


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("V", [1000, 4096, 50257])
def test_sample_small_vocab(cuda, dtype, V):
    x, tk, tp, T, noise = o.make_sampling_inputs(B=24, V=V, seed=11, dtype=dtype)
    tk = np.minimum(tk, V).astype(np.int32)
    T[1] = 1e-6
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, _ = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_sample_decode_configuration(cuda, dtype):
    # benchmark configuration 3 at reduced batch: bf16 [*, 128256], top_k 1..1024 with 10 % disabled
    x, tk, tp, T, noise = o.make_sampling_inputs(B=48, V=128256, seed=2, dtype=dtype)
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, status = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags)
    assert np.array_equal(status & 1 != 0, tk == 0)  # only the top-k-disabled rows take the general path
    assert (status & 2 == 0).all()


def test_sample_decode_configuration_full_batch(cuda):
    x, tk, tp, T, noise = o.make_sampling_inputs(B=256, V=128256, seed=2, dtype="bf16")
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, _ = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.95)
    # size-independent properties: the token lies in the row's top-k set and is repeatable
    xf = x.astype(np.float32)
    for b in range(256):
        if tk[b] > 0:
            kth = np.partition(xf[b], -int(tk[b]))[-int(tk[b])]
            assert xf[b, got[b]] >= kth
    again, _ = _run(cuda, x, tk, tp, T, noise=noise)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_sample_general_path_cases(cuda, dtype):
    B, V = 20, 60000
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=21, dtype=dtype)
    tk[:] = [0, 0, 2000, 5000, V, V + 5, -1, 1500, 30000, 59999, 0, 0, 1025, 0, 0, 0, 0, 0, 0, 0]
    tp[:8] = [0.3, 0.999, 0.9, 0.5, 0.7, 0.95, 0.2, 1.0]
    T[10] = 1e-7
    if dtype == "bf16":
        x[11] = (np.arange(V) % 7).astype(np.float32)     # heavy ties everywhere
        x[12] = x[12].astype(np.float32).round()            # top-k boundary cuts through a tie group
        x[13] = -np.abs(x[13].astype(np.float32))           # all-negative row (log-prob like)
    else:
        x[11] = (np.arange(V) % 7).astype(np.float32)
        x[12] = x[12].round()
        x[13] = -np.abs(x[13])
    x[14, 100:] = -np.inf                                   # almost everything masked
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, status = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.7)
    assert (status[[0, 1, 3]] & 1).all()   # no top-k, or one above the candidate path's limit


def test_sample_rows_without_top_k_in_a_large_batch(cuda):
    # Large batches send the rows without top-k to the cluster kernel (the row resident in shared
    # memory).  Flat rows push the top-p boundary below the first histogram window, into the
    # negative values, so the window-by-window search is exercised, next to ties, masks and top_p = 1.
    B, V = 320, 32768
    rng = np.random.default_rng(5)
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=31, dtype="bf16")
    tk[:] = rng.integers(1, 600, B)
    wide = np.arange(B) % 2 == 0
    tk[wide] = 0
    scale = np.where(np.arange(B) % 4 == 0, 0.05, 1.0).astype(np.float32)[:, None]   # every other wide row is flat
    x = (x.astype(np.float32) * scale).astype(o.bfloat16)
    tp[:] = rng.uniform(0.3, 0.98, B).astype(np.float32)
    tp[8] = 1.0
    tp[12] = 0.9999
    x[16] = (np.arange(V) % 5).astype(np.float32).astype(o.bfloat16)        # five value groups
    x[20] = (-np.abs(x[20].astype(np.float32)) - 1.0).astype(o.bfloat16)    # all negative
    x[24, 50:] = -np.inf                                                    # almost everything masked
    x[28] = 0.0                                                             # a single value group
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, status = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.8)
    assert (status[wide] & 1).all() and (status & 2 == 0).all()
    assert (~flags[(np.arange(B) % 4 == 0)]).mean() > 0.5   # the flat rows are really checked


def test_sample_fast_path_overflow_falls_back(cuda):
    # ascending rows overflow the candidate list; the general kernel must answer them
    V = 70000
    x = np.tile(np.linspace(-8, 8, V, dtype=np.float32), (6, 1)).astype(o.bfloat16)
    tk = np.array([5, 50, 500, 1000, 64, 1], np.int32)
    tp = np.array([0.9, 0.8, 0.99, 0.5, 1.0, 0.9], np.float32)
    T = np.array([1.0, 0.7, 1.3, 0.9, 1.1, 1.0], np.float32)
    noise = np.random.default_rng(0).random((6, V), dtype=np.float32)
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, status = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.5)
    assert (status & 2 == 0).all()  # no bounded wait gave up


def test_sample_with_threefry_key_and_row_offset(cuda):
    x, tk, tp, T, _ = o.make_sampling_inputs(B=16, V=32000, seed=31, dtype="bf16")
    key = (0xDEADBEEF, 12345)
    exp, flags = o.sample(x, tk, tp, T, rng_key=key, dim0_offset=0, return_flags=True)
    got, _ = _run(cuda, x, tk, tp, T, key=key)
    _assert_tokens(got, exp, flags)
    # a batch shard: rows 8..15 sampled alone with dim0_offset=8 reproduce the unsharded tokens
    got2, _ = _run(cuda, x[8:], tk[8:], tp[8:], T[8:], key=key, dim0_offset=8)
    _assert_tokens(got2, exp[8:], flags[8:], min_checked=0.7)


def test_public_sample_entry_point(cuda):
    x, tk, tp, T, noise = o.make_sampling_inputs(B=8, V=20000, seed=41, dtype="bf16")
    md = sampling.SamplingMetadata(top_k=to_dev(tk, cuda), top_p=to_dev(tp, cuda), temperature=to_dev(T, cuda))
    tok = sampling.sample(None, to_dev(x, cuda), md, noise=to_dev(noise, cuda))
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    _assert_tokens(to_np(tok), exp, flags, min_checked=0.7)
    assert tok.dtype == torch.int32 and tok.shape == (8,)
    with pytest.raises(ValueError):
        sampling.sample(None, to_dev(x, cuda), md)  # neither key nor noise


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("k", [128, 64, 1000])
def test_top_p_and_sample(cuda, dtype, k):
    V, B = 32000, 16
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=51, dtype=dtype)
    tk = np.clip(tk, 1, k).astype(np.int32)
    T[2] = 0.0
    vals, idx = o.top_dynamic_k(x, tk, k, replace_val=-1e12)
    exp, flags = o.top_p_and_sample(vals, idx, tp, T, vocab_size=V, replace_val=-1e12, noise=noise,
                                    return_flags=True)
    got = sampling.top_p_and_sample(to_dev(vals, cuda), to_dev(idx, cuda), None, to_dev(tp, cuda), to_dev(T, cuda),
                                    vocab_size=V, replace_val=-1e12, noise=to_dev(noise, cuda))
    _assert_tokens(to_np(got), exp, flags, min_checked=0.7)
    key = (7, 8)
    exp2, flags2 = o.top_p_and_sample(vals, idx, tp, T, vocab_size=V, replace_val=-1e12, rng_key=key, dim0_offset=3,
                                      return_flags=True)
    got2 = sampling.top_p_and_sample(to_dev(vals, cuda), to_dev(idx, cuda), key, to_dev(tp, cuda), to_dev(T, cuda),
                                     vocab_size=V, replace_val=-1e12, dim0_offset=3)
    _assert_tokens(to_np(got2), exp2, flags2, min_checked=0.7)
    # and the two-stage composition equals the fused sampler (both are the reference's `sample`)
    fused, _ = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(fused, exp, flags, min_checked=0.7)


def test_top_p_mask(cuda):
    rng = np.random.default_rng(61)
    x = -np.sort(-rng.standard_normal((128, 24)).astype(np.float32) * 3, axis=0)
    p = rng.uniform(0.05, 0.999, 24).astype(np.float32)
    got = to_np(sampling.top_p_mask(topk_logits=to_dev(x, cuda), p=to_dev(p, cuda), replace_val=-1e12, axis=0))
    exp = o.top_p_mask(x, p, -1e12)
    e = np.exp(x.astype(np.float64) - x[:1])
    cs = np.cumsum(e / e.sum(0), axis=0)
    near = np.abs(cs - p[None, :]).min(axis=0) < TOL_NEAR_THRESHOLD
    assert np.array_equal(got[:, ~near], exp[:, ~near]) and (~near).sum() >= 20


@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_vocab_sharded_pipeline_on_one_device(cuda, n_shards):
    # the per-shard stage, a concatenation standing in for the all-gather, and the merge stage
    B, V = 32, 151936
    x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=4, dtype="bf16")
    tk = np.random.default_rng(1).integers(1, 51, B).astype(np.int32)
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    vl = V // n_shards
    dx, dn = to_dev(x, cuda), to_dev(noise, cuda)
    blocks = [ops.shard_candidates(dx[:, s * vl:(s + 1) * vl].contiguous(), s * vl, 50,
                                   noise_shard=dn[:, s * vl:(s + 1) * vl].contiguous()) for s in range(n_shards)]
    # stage 1 against the oracle's stage 1
    ev, ei, en = o.shard_candidates(x[:, :vl], 0, 50, noise[:, :vl])
    b0 = blocks[0]
    assert np.array_equal(to_np(b0[0]), ev) and np.array_equal(to_np(b0[1].view(torch.int32)), ei)
    assert np.array_equal(to_np(b0[2]), en)
    got = ops.merge_and_sample(torch.stack(blocks), to_dev(tk, cuda), to_dev(tp, cuda), to_dev(T, cuda))
    _assert_tokens(to_np(got), exp, flags, min_checked=0.7)
    assert np.array_equal(exp, o.sample_vocab_sharded(x, n_shards, tk, tp, T, noise))


def test_vocab_sharded_entry_point_single_rank(cuda):
    B, V = 8, 40000
    x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=5, dtype="bf16")
    md = sampling.SamplingMetadata(top_k=to_dev(tk, cuda), top_p=to_dev(tp, cuda), temperature=to_dev(T, cuda))
    got = sampling.sample_vocab_sharded(None, to_dev(x, cuda), md, noise_shard=to_dev(noise, cuda), k_cand=50)
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    _assert_tokens(to_np(got), exp, flags, min_checked=0.7)


@pytest.mark.parametrize("seed", [31, 32, 33])
def test_sample_f32_top_k_between_1025_and_2048(cuda, seed):
    # more rows than SMs, every row with a top_k that the candidate path serves but that exceeds
    # 2 x (threads per CTA) candidates in the tail
    B, V = 160, 40000
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=seed, dtype="f32")
    tk[:] = np.random.default_rng(seed).integers(1025, 2049, B).astype(np.int32)
    tk[:4] = [1025, 2048, 2047, 1536]
    tp[::3] = 1.0   # the whole top-k set is kept: the tail walks all of its candidates
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, status = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.6)   # top_p == 1 sits on the threshold by construction
    assert (status & 2 == 0).all()


def test_sample_bf16_top_k_2000_over_few_finite_logits(cuda):
    B, V = 12, 50000
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=41, dtype="bf16")
    rng = np.random.default_rng(41)
    xf = x.astype(np.float32)
    for b in range(B):
        keep = rng.choice(V, size=100, replace=False)
        m = np.full(V, -np.inf, np.float32)
        m[keep] = xf[b, keep]
        xf[b] = m
    x = xf.astype(x.dtype)
    tk[:] = 2000
    tp[:] = np.linspace(0.5, 1.0, B).astype(np.float32)
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    got, _ = _run(cuda, x, tk, tp, T, noise=noise)
    _assert_tokens(got, exp, flags, min_checked=0.7)
    assert np.isfinite(x.astype(np.float32)[np.arange(B), got]).all()


@pytest.mark.parametrize("top_k", [0, 1500, 2048])
def test_merge_and_sample_with_more_than_1024_candidates(cuda, top_k):
    # 8 shards x 256 candidates: with top-k disabled (or large) the tail walks all 2048 of them
    B, V, n_shards, k_cand = 16, 65536, 8, 256
    x, _, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=6, dtype="bf16")
    tk = np.full(B, top_k, np.int32)
    tp[::4] = 0.9999   # nearly the whole candidate set is kept: the tail walks all of it
    vl = V // n_shards
    parts = [o.shard_candidates(x[:, s * vl:(s + 1) * vl], s * vl, k_cand, noise[:, s * vl:(s + 1) * vl])
             for s in range(n_shards)]
    cv, ci, cn = (np.concatenate([p[i] for p in parts], axis=1) for i in range(3))
    exp, flags = o.merge_and_sample(cv, ci, cn, tk, tp, T, return_flags=True)
    dx, dn = to_dev(x, cuda), to_dev(noise, cuda)
    blocks = [ops.shard_candidates(dx[:, s * vl:(s + 1) * vl].contiguous(), s * vl, k_cand,
                                   noise_shard=dn[:, s * vl:(s + 1) * vl].contiguous()) for s in range(n_shards)]
    got = ops.merge_and_sample(torch.stack(blocks), to_dev(tk, cuda), to_dev(tp, cuda), to_dev(T, cuda))
    _assert_tokens(to_np(got), exp, flags, min_checked=0.7)


@pytest.mark.parametrize("dtype,v_local,k", [("bf16", 18992, 50), ("f32", 20000, 128), ("bf16", 37984, 50), ("bf16", 700, 50)])
def test_shard_candidates_of_many_short_rows(cuda, dtype, v_local, k):
    # the shard's top-k by (value desc, index asc), global token ids, the noise at those tokens, on rows that
    # defeat a sampled threshold (one value only, ascending, fewer finite values than k, NaNs)
    B = 300
    x, _, _, _, noise = o.make_sharded_inputs(B=B, V=v_local, seed=12, dtype=dtype)
    xf = x.astype(np.float32)
    xf[0] = 1.5                                        # one value only: a tie group larger than any list
    xf[1] = np.round(xf[1])                            # heavy ties around the k-th value
    xf[2] = np.arange(v_local, dtype=np.float32) / 64   # ascending: the sample sees only the smallest elements
    xf[3] = -np.arange(v_local, dtype=np.float32) / 64  # descending
    xf[4, 40:] = -np.inf                               # fewer finite values than k
    xf[5, ::3] = np.nan
    x = xf.astype(x.dtype)
    ev, ei, en = o.shard_candidates(x, 1000, k, noise)
    got = ops.shard_candidates(to_dev(x, cuda), 1000, k, noise_shard=to_dev(noise, cuda))
    gv, gi, gn = to_np(got[0]), to_np(got[1].view(torch.int32)), to_np(got[2])
    assert np.array_equal(gi, ei)
    assert np.array_equal(gv, ev, equal_nan=True) and np.array_equal(gn, en)


@pytest.mark.parametrize("B", [1, 2, 5, 600, 2048])
def test_streaming_path_row_counts(cuda, B):
    # fewer items than CTAs, more rows than finish CTAs resident at a time, and rows of every class in one batch;
    # the oracle checks a sample of the rows, repeat calls check determinism of the rest
    V = 32768
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=50 + B, dtype="bf16")
    tk[::7] = 0
    if B > 3:
        tp[3] = 1.0
        tk[3] = 0       # no filter at all: the whole-row routine
        T[4] = 0.0      # greedy
    args = [to_dev(a, cuda) for a in (x, tk, tp, T)]
    dn = to_dev(noise, cuda)
    tok, status = ops.sample(*args, noise=dn, return_status=True)
    got = to_np(tok).copy()
    assert (to_np(status) & 2 == 0).all()
    sel = np.unique(np.concatenate([np.arange(min(B, 8)), np.random.default_rng(B).integers(0, B, 40)]))
    exp, flags = o.sample(x[sel], tk[sel], tp[sel], T[sel], noise=noise[sel], return_flags=True)
    assert not ((got[sel] != exp) & ~flags).any()
    for _ in range(2):
        again, _ = ops.sample(*args, noise=dn, return_status=True)
        assert np.array_equal(to_np(again), got)
