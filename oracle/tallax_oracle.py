"""CPU restatement (NumPy) of tallax's row-wise hot path.  TEST INFRASTRUCTURE ONLY.

This module is the correctness checker for the CUDA library.  Nothing in the
product package may import it; only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark do.

PARITY STATUS.  The reference is pure JAX/Pallas-TPU, JAX is not installable here and the
reference stores no golden vectors (its tests recompute every expectation through jax).
What pins this oracle:
  * threefry2x32: the Random123 known-answer vectors that JAX's own tests use (`THREEFRY_KAT`);
  * key transform, cumsum, gather (with out-of-range indices), max_arrays, indexed uniform
    noise, top_p_mask, top_p_and_sample (token ids) and the sparse categorical draw: outputs
    of the REFERENCE'S OWN value-level functions, run from the reference checkout with
    jax.numpy mapped onto NumPy (tests/golden/make_golden.py, fixtures in tests/golden/,
    checked by tests/test_golden.py);
  * sort and top-k: "parity unpinned" against reference outputs (their reference code only
    exists as Pallas kernels); they are defined as the NumPy twins of the XLA functions the
    reference's tests compare with (stable lexicographic sort; descending stable argsort).

Each function cites the reference file:line it restates (paths inside the
reference project).
"""
from __future__ import annotations

import numpy as np

try:  # bf16 in numpy
    import ml_dtypes

    bfloat16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    bfloat16 = None

F32_TINY = np.finfo(np.float32).tiny
SAMPLING_EPS = 1e-5  # tallax/_src/sampling.py:22
NEAR_THRESHOLD = 1e-6  # rows whose cumulative mass is this close to top_p are exempt


# ----------------------------------------------------------------------------
# key transforms                                   tallax/_src/utils.py:139-200
# ----------------------------------------------------------------------------
def sortable_key_u32(x: np.ndarray) -> np.ndarray:
    """Order-preserving map of a 32-bit (or narrower) array to uint32.

    float: NaN -> one canonical key above +inf, -0 -> +0 (utils.py:139-147), then
    the sign-flip trick (utils.py:186-195, restated on unsigned ints).
    int32: offset binary.  bf16/f16 are widened to f32 first (exact).
    """
    x = np.asarray(x)
    if x.dtype == np.int32:
        return (x.view(np.uint32) ^ np.uint32(0x80000000)).astype(np.uint32)
    if x.dtype == np.uint32:
        return x.copy()
    if x.dtype.kind == "i" or x.dtype.kind == "u" or x.dtype.kind == "b":
        return sortable_key_u32(x.astype(np.int32))
    xf = np.ascontiguousarray(x.astype(np.float32))
    b = xf.view(np.uint32).copy()
    b[xf == 0] = 0
    neg = (b >> np.uint32(31)).astype(bool)
    k = np.where(neg, ~b, b | np.uint32(0x80000000)).astype(np.uint32)
    k[np.isnan(xf)] = np.uint32(0xFFFFFFFF)
    return k


def key_u32_to_f32(k: np.ndarray) -> np.ndarray:
    """Inverse of `sortable_key_u32` for float keys (utils.py:198-200)."""
    k = np.asarray(k, dtype=np.uint32)
    pos = (k >> np.uint32(31)).astype(bool)
    b = np.where(pos, k & np.uint32(0x7FFFFFFF), ~k).astype(np.uint32)
    return b.view(np.float32)


def _canon(x: np.ndarray) -> np.ndarray:
    """What a float key looks like after a round trip through the key domain."""
    if np.asarray(x).dtype.kind != "f" and np.asarray(x).dtype != bfloat16:
        return np.asarray(x)
    return key_u32_to_f32(sortable_key_u32(x)).astype(np.asarray(x).dtype)


# ----------------------------------------------------------------------------
# sort                         tallax/_src/sort.py:768-929, oracle sort.py:937-969
# ----------------------------------------------------------------------------
def sort(operands, num_keys, is_stable=False, return_argsort=False, descending=False):
    """Row-wise multi-operand sort; the definition `xla_equivalent_sort` gives.

    Keys are compared lexicographically in the canonical key domain; ties keep
    ascending column order (also when `descending`), which is the stable
    definition and one valid answer for the unstable variants.  Key outputs are
    returned canonicalised (-0 -> +0, NaN -> canonical NaN) as in sort.py:834-839.
    """
    ops = [np.asarray(o) for o in (operands if isinstance(operands, (list, tuple)) else [operands])]
    shape = ops[0].shape
    if any(o.shape != shape for o in ops):
        raise ValueError("Inputs must all have the same shape")
    if len(shape) != 2:
        raise ValueError("Only 2D inputs supported")
    rows, n = shape
    perm = np.empty((rows, n), dtype=np.int64)
    keys = [sortable_key_u32(o).astype(np.int64) for o in ops[:num_keys]]
    if descending:
        keys = [-k for k in keys]
    col = np.arange(n)
    for r in range(rows):
        # np.lexsort: last key is the primary one
        perm[r] = np.lexsort([col] + [k[r] for k in keys[::-1]])
    outs = []
    for i, o in enumerate(ops):
        g = np.take_along_axis(o, perm, axis=1)
        if i < num_keys:
            g = _canon(g)
        outs.append(g)
    if return_argsort:
        outs.append(perm.astype(np.int32))
    return tuple(outs)


def argsort(x, descending=False):
    return sort([x], 1, is_stable=True, return_argsort=True, descending=descending)[1]


# ----------------------------------------------------------------------------
# top-k                    tallax/_src/top_k.py:385-567, bitonic_top_k.py:343-402
# ----------------------------------------------------------------------------
def top_k(x, k):
    """Descending top-k of each row, ties broken by lower index.

    Values keep the input dtype and bits (top_k.py:509-513 returns slices of
    the input values); indices are int32.
    """
    x = np.asarray(x)
    key = sortable_key_u32(x).astype(np.int64)
    order = np.argsort(-key, axis=1, kind="stable")[:, :k]
    return np.take_along_axis(x, order, axis=1), order.astype(np.int32)


def top_dynamic_k(x, k, max_k, replace_val=None):
    """Per-row k (top_k.py:365-369): positions >= k[row] hold `replace_val`."""
    vals, idx = top_k(x, max_k)
    if replace_val is not None:
        kk = np.broadcast_to(np.asarray(k), (x.shape[0],))
        mask = np.arange(max_k)[None, :] >= kk[:, None]
        vals = vals.copy()
        vals[mask] = np.asarray(replace_val).astype(vals.dtype)
    return vals, idx


def bitonic_top_k(operands, k=128, num_keys=1):
    """Multi-operand descending top-k (bitonic_top_k.py:343-402).

    First `num_keys` operands are lexicographic keys; every operand is permuted
    alike.  Tie order in the reference is network order; lower column first here.
    """
    ops = [np.asarray(o) for o in operands]
    outs = sort(ops, num_keys, is_stable=True, descending=True, return_argsort=True)
    perm = outs[-1][:, :k].astype(np.int64)
    return tuple(np.take_along_axis(o, perm, axis=1) for o in ops)


def max_arrays(operands, num_keys, axis):
    """Lexicographic arg-max carrying payloads (bitonic_top_k.py:43-97)."""
    ops = [np.asarray(o) for o in operands]
    if axis == 0:
        ops = [o.T for o in ops]
    outs = bitonic_top_k(ops, k=1, num_keys=num_keys)
    return [o[:, 0] for o in outs]


def topk_recall(approx_idx, exact_idx):
    """Mean over rows of |approx ∩ exact| / k (yardstick in benchmarks/top_k_benchmark.py:45-46)."""
    r = [len(set(a.tolist()) & set(e.tolist())) / len(e) for a, e in zip(approx_idx, exact_idx)]
    return float(np.mean(r))


# ----------------------------------------------------------------------------
# gather                                           tallax/_src/gather.py:11-45
# ----------------------------------------------------------------------------
def take_along_axis(values, indices, axis):
    """`np.take_along_axis` for in-range indices; out-of-range or negative -> 0.

    The reference's accumulators start at zero and a range mask never fires for
    an index outside [0, n) (gather.py:17-20,28,35).
    """
    values = np.asarray(values)
    indices = np.asarray(indices)
    n = values.shape[axis]
    ok = (indices >= 0) & (indices < n)
    safe = np.where(ok, indices, 0).astype(np.int64)
    out = np.take_along_axis(values, safe, axis=axis)
    return np.where(ok, out, np.zeros((), dtype=values.dtype)).astype(values.dtype)


# ----------------------------------------------------------------------------
# cumsum                                           tallax/_src/cumsum.py:21-63
# ----------------------------------------------------------------------------
def cumsum(arr, axis, reverse=False, accum=None):
    """Inclusive prefix sum along `axis`, optionally reversed.

    Integer: exact (wraps like int32).  Float: the reference's own tolerance is
    rtol 1e-3 / atol 1e-6 against lax.cumsum (tests/cumsum_test.py:31); pass
    `accum=np.float64` for a tight yardstick.
    """
    a = np.asarray(arr)
    if reverse:
        a = np.flip(a, axis=axis)
    out = np.cumsum(a, axis=axis, dtype=accum if accum is not None else a.dtype)
    if reverse:
        out = np.flip(out, axis=axis)
    return np.ascontiguousarray(out)


# ----------------------------------------------------------------------------
# counter-based noise                     tallax/_src/sparse_random.py:7-94
# ----------------------------------------------------------------------------
# Random123 known-answer vectors for Threefry-2x32, 20 rounds
# (key, counter) -> output; the same three vectors JAX's random tests use.
THREEFRY_KAT = [
    ((0x00000000, 0x00000000), (0x00000000, 0x00000000), (0x6B200159, 0x99BA4EFE)),
    ((0xFFFFFFFF, 0xFFFFFFFF), (0xFFFFFFFF, 0xFFFFFFFF), (0x1CB996FC, 0xBB002BE7)),
    ((0x13198A2E, 0x03707344), (0x243F6A88, 0x85A308D3), (0xC4923A9C, 0x483DF7A0)),
]

_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))


def threefry2x32(key, x0, x1):
    """Threefry-2x32 with 20 rounds (the `threefry2x32_p` primitive that
    sparse_random.py:54 binds), restated from the published algorithm."""
    k0 = np.uint32(key[0])
    k1 = np.uint32(key[1])
    k2 = np.uint32(k0 ^ k1 ^ np.uint32(0x1BD11BDA))
    ks = (k0, k1, k2)
    x0 = np.asarray(x0, dtype=np.uint32).copy()
    x1 = np.asarray(x1, dtype=np.uint32).copy()
    with np.errstate(over="ignore"):
        x0 = x0 + ks[0]
        x1 = x1 + ks[1]
        for blk in range(5):
            for r in _ROT[blk % 2]:
                x0 = x0 + x1
                x1 = (x1 << np.uint32(r)) | (x1 >> np.uint32(32 - r))
                x1 = x1 ^ x0
            x0 = x0 + ks[(blk + 1) % 3]
            x1 = x1 + ks[(blk + 2) % 3] + np.uint32(blk + 1)
    return x0, x1


def bits_to_uniform(bits):
    """uint32 bits -> f32 in [0,1) by the mantissa trick (sparse_random.py:7-41)."""
    b = (np.asarray(bits, dtype=np.uint32) >> np.uint32(9)) | np.uint32(0x3F800000)
    return b.view(np.float32) - np.float32(1.0)


def sparse_random_uniform(key, indices, dim1_size, minval=0.0, maxval=1.0):
    """Uniform noise at (i0, i1) of a virtual dense [*, dim1_size] array
    (sparse_random.py:43-64): counter = (0, i0*dim1_size + i1), bits = x0 ^ x1."""
    i0, i1 = (np.asarray(i) for i in indices)
    with np.errstate(over="ignore"):
        lo = (i0.astype(np.int64) * int(dim1_size) + i1.astype(np.int64)).astype(np.uint32)
    b0, b1 = threefry2x32(key, np.zeros_like(lo), lo)
    f = bits_to_uniform(b0 ^ b1)
    mn = np.float32(minval)
    mx = np.float32(maxval)
    return np.maximum(mn, f * (mx - mn) + mn).astype(np.float32)


def dense_uniform(key, shape, dim0_offset=0):
    """The dense [B, V] tensor of which `sparse_random_uniform` reads entries, with
    the sampler's range [tiny, 1) (sparse_random.py:75-82)."""
    b, v = shape
    i0 = np.arange(b, dtype=np.int64)[:, None] + dim0_offset
    i1 = np.arange(v, dtype=np.int64)[None, :]
    return sparse_random_uniform(key, (np.broadcast_to(i0, shape), np.broadcast_to(i1, shape)), v,
                                 minval=F32_TINY, maxval=1.0)


def gumbel_from_uniform(u):
    """g = -log(-log(max(u, tiny))) (sparse_random.py:75-84), evaluated in f64 and
    rounded to f32 once so that CPU and GPU agree bit for bit."""
    u = np.maximum(np.asarray(u, dtype=np.float32), np.float32(F32_TINY)).astype(np.float64)
    with np.errstate(divide="ignore"):
        return (-np.log(-np.log(u))).astype(np.float32)


# ----------------------------------------------------------------------------
# candidate-level sampler                     tallax/_src/sampling.py:25-115
# ----------------------------------------------------------------------------
def top_p_mask(topk_logits, p, replace_val, axis=0):
    """Literal restatement of sampling.py:25-62 on (k, B) f32 candidates sorted
    descending along axis 0, including the out-of-range gather -> 0.0 quirk."""
    if axis != 0:
        raise NotImplementedError("topp_mask only supports axis=0")
    x = np.asarray(topk_logits, dtype=np.float32)
    e = np.exp(x - x[:1, :])
    probs = e / e.sum(axis=0, keepdims=True)
    cs = cumsum(probs, 0)
    t = (cs < np.asarray(p, dtype=np.float32)[None, :]).sum(0, keepdims=True)
    thr = take_along_axis(x, np.broadcast_to(t, x.shape), 0)
    return np.where(x >= thr, x, np.float32(replace_val)).astype(np.float32)


def _row_sample(xs, tok, u, p, T, n_valid):
    """Shared tail of the samplers for ONE row.

    xs: f32 candidates sorted by (value desc, token asc); only the first
    `n_valid` are in the top-k set.  tok: their token ids.  u: their uniform
    noise.  Returns (token, near_threshold_flag).
    """
    xs = xs[:n_valid].astype(np.float32)
    tok = tok[:n_valid]
    u = u[:n_valid]
    if np.float32(T) < np.float32(SAMPLING_EPS):  # sampling.py:112-115
        return int(tok[0]), False
    e = np.exp(xs.astype(np.float64) - np.float64(xs[0]))
    cs = np.cumsum(e / e.sum())
    pf = np.float64(np.float32(p))
    near = bool(np.min(np.abs(cs - pf)) < NEAR_THRESHOLD)
    t = min(int((cs < pf).sum()), n_valid - 1)  # sampling.py:52; clamp replaces the OOB quirk
    keep = xs >= xs[t]  # ties at the threshold all kept, sampling.py:53-60
    y = (xs / np.float32(T)).astype(np.float32) + gumbel_from_uniform(u)  # :97, sparse_random.py:84-86
    y = np.where(keep, y, -np.inf).astype(np.float32)
    best = np.flatnonzero(y == y.max())
    return int(tok[best].min()), near  # exact y ties -> lowest token id (dense categorical's rule)


def top_p_and_sample(topk_logits, topk_idx, top_p, temperature, *, vocab_size, replace_val,
                     rng_key=None, noise=None, dim0_offset=0, return_flags=False):
    """sampling.py:65-115 on [B, k] candidates already sorted descending, with
    positions beyond the row's top-k already set to `replace_val` by the caller
    (sampling.py:277-281 / top_k.py:365-369).

    Noise: either `rng_key` (two uint32, threefry counter (b+dim0_offset)*V + token)
    or `noise`, the dense uniform tensor [B_total, V] indexed the same way.
    """
    raw = np.asarray(topk_logits)
    x = raw.astype(np.float32)
    rep = np.asarray(replace_val).astype(raw.dtype).astype(np.float32)  # as stored in the candidates' dtype
    idx = np.asarray(topk_idx).astype(np.int64)
    B, k = x.shape
    top_p = np.broadcast_to(np.asarray(top_p, dtype=np.float32), (B,))
    temperature = np.broadcast_to(np.asarray(temperature, dtype=np.float32), (B,))
    out = np.empty(B, dtype=np.int32)
    flags = np.zeros(B, dtype=bool)
    for b in range(B):
        valid = x[b] != rep
        n_valid = int(valid.sum()) if valid.any() else 1
        if noise is not None:
            u = np.asarray(noise)[b + dim0_offset, idx[b]]
        else:
            u = sparse_random_uniform(rng_key, (np.full(k, b + dim0_offset), idx[b]), vocab_size,
                                      minval=F32_TINY, maxval=1.0)
        out[b], flags[b] = _row_sample(x[b], idx[b], u, top_p[b], temperature[b], n_valid)
    return (out, flags) if return_flags else out


# ----------------------------------------------------------------------------
# dense fused sampler          tallax/_src/sampling.py:271-343 (`sample`)
# ----------------------------------------------------------------------------
def sample(logits, top_k_, top_p, temperature, *, noise=None, rng_key=None, dim0_offset=0,
           return_flags=False):
    """logits [B, V] -> token ids [B].

    Per row: order = stable descending argsort of f32(logits); K = top_k if
    0 < top_k < V else V (extension: the reference caps K at 128 and has no
    'disabled' value); softmax over the K candidates on UNSCALED logits
    (sampling.py:45-46), f64 cumulative mass, threshold with ties kept
    (:52-60), divide by temperature (:97), add Gumbel noise read at the
    candidates' tokens (:101-111), arg-max; temperature < 1e-5 -> greedy (:112-115).
    """
    x = np.asarray(logits).astype(np.float32)
    B, V = x.shape
    kk = np.broadcast_to(np.asarray(top_k_, dtype=np.int64), (B,))
    top_p = np.broadcast_to(np.asarray(top_p, dtype=np.float32), (B,))
    temperature = np.broadcast_to(np.asarray(temperature, dtype=np.float32), (B,))
    key = sortable_key_u32(x).astype(np.int64)
    out = np.empty(B, dtype=np.int32)
    flags = np.zeros(B, dtype=bool)
    for b in range(B):
        K = int(kk[b]) if 0 < kk[b] < V else V
        if K < V:
            part = np.argpartition(-key[b], K - 1)[:K]
            vk = key[b][part].min()
            # all strictly greater, then lowest-indexed ties
            gt = np.flatnonzero(key[b] > vk)
            eq = np.flatnonzero(key[b] == vk)[: K - len(gt)]
            cand = np.concatenate([gt, eq])
        else:
            cand = np.arange(V)
        order = cand[np.lexsort((cand, -key[b][cand]))]
        if noise is not None:
            u = np.asarray(noise)[b + dim0_offset, order]
        else:
            u = sparse_random_uniform(rng_key, (np.full(len(order), b + dim0_offset), order), V,
                                      minval=F32_TINY, maxval=1.0)
        out[b], flags[b] = _row_sample(x[b][order], order, u, top_p[b], temperature[b], K)
    return (out, flags) if return_flags else out


def sample_two_stage(logits, top_k_, top_p, temperature, *, noise=None, rng_key=None, max_k=128):
    """The literal two-stage composition of sampling.py:331-343 for 1 <= top_k <= max_k:
    top-`max_k` with per-row masking, then `top_p_and_sample`."""
    REPLACE = -1e12
    x = np.asarray(logits).astype(np.float32)
    vals, idx = top_dynamic_k(x, top_k_, max_k, replace_val=REPLACE)
    return top_p_and_sample(vals, idx, top_p, temperature, vocab_size=x.shape[1], replace_val=REPLACE,
                            rng_key=rng_key, noise=noise)


# ----------------------------------------------------------------------------
# vocab-sharded sampler                      tallax/_src/sampling.py:300-321
# ----------------------------------------------------------------------------
def shard_candidates(logits_shard, col_offset, k_cand, noise_shard):
    """One vocab shard's contribution: its local top-`k_cand` (value f32, GLOBAL
    token id, the uniform noise at that token), sampling.py:306-311."""
    x = np.asarray(logits_shard).astype(np.float32)
    vals, idx = top_k(x, k_cand)
    u = np.take_along_axis(np.asarray(noise_shard), idx.astype(np.int64), axis=1)
    return vals, (idx + col_offset).astype(np.int32), u.astype(np.float32)


def merge_and_sample(cand_vals, cand_idx, cand_noise, top_k_, top_p, temperature, return_flags=False):
    """After the all-gather (sampling.py:313): merge the n_shards*k' candidates by
    (value desc, global token asc), keep the row's top-k, then the sampler tail."""
    v = np.asarray(cand_vals, dtype=np.float32)
    B, M = v.shape
    kk = np.broadcast_to(np.asarray(top_k_, dtype=np.int64), (B,))
    top_p = np.broadcast_to(np.asarray(top_p, dtype=np.float32), (B,))
    temperature = np.broadcast_to(np.asarray(temperature, dtype=np.float32), (B,))
    key = sortable_key_u32(v).astype(np.int64)
    out = np.empty(B, dtype=np.int32)
    flags = np.zeros(B, dtype=bool)
    for b in range(B):
        order = np.lexsort((np.asarray(cand_idx)[b], -key[b]))
        K = M if kk[b] <= 0 or kk[b] > M else int(kk[b])   # top_k <= 0: disabled, as in `sample`
        out[b], flags[b] = _row_sample(v[b][order], np.asarray(cand_idx)[b][order].astype(np.int64),
                                       np.asarray(cand_noise)[b][order], top_p[b], temperature[b], K)
    return (out, flags) if return_flags else out


def sample_vocab_sharded(logits, n_shards, top_k_, top_p, temperature, noise, return_flags=False):
    """Emulates the n-shard pipeline on one host; must equal `sample` on the
    unsharded logits whenever 1 <= top_k <= V/n_shards (sampling.py:248's intent)."""
    x = np.asarray(logits)
    B, V = x.shape
    assert V % n_shards == 0
    vl = V // n_shards
    k_cand = int(np.max(np.broadcast_to(np.asarray(top_k_), (B,))))
    parts = [shard_candidates(x[:, s * vl:(s + 1) * vl], s * vl, k_cand, np.asarray(noise)[:, s * vl:(s + 1) * vl])
             for s in range(n_shards)]
    cv, ci, cn = (np.concatenate([p[i] for p in parts], axis=1) for i in range(3))
    return merge_and_sample(cv, ci, cn, top_k_, top_p, temperature, return_flags=return_flags)


# ----------------------------------------------------------------------------
# synthetic workloads with the benchmark configurations' shapes and distributions
# (NumPy Philox streams stand in for the jax.random streams the configs name)
# ----------------------------------------------------------------------------
def make_sampling_inputs(B=256, V=128256, seed=2, sigma=3.0, dtype="bf16", spikes=8):
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.standard_normal((B, V), dtype=np.float32) * np.float32(sigma)
    for b in range(B):
        cols = rng.choice(V, size=min(spikes, V), replace=False)
        x[b, cols] += np.float32(10.0)
    if dtype == "bf16":
        x = x.astype(bfloat16)
    temperature = rng.uniform(0.5, 1.5, size=B).astype(np.float32)
    top_k_ = rng.integers(1, 1025, size=B).astype(np.int32)
    top_k_[rng.random(B) < 0.1] = 0
    top_p = rng.uniform(0.6, 1.0, size=B).astype(np.float32)
    noise = rng.random((B, V), dtype=np.float32)
    return x, top_k_, top_p, temperature, noise


def make_sharded_inputs(B=1024, V=151936, seed=4, dtype="bf16"):
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.standard_normal((B, V), dtype=np.float32) * np.float32(2.0)
    bias = (4.0 * np.arange(1, V + 1, dtype=np.float64) ** -1.1).astype(np.float32)
    for b in range(B):
        x[b, rng.permutation(V)] += bias
    if dtype == "bf16":
        x = x.astype(bfloat16)
    noise = rng.random((B, V), dtype=np.float32)
    return x, np.full(B, 50, np.int32), np.full(B, 0.95, np.float32), np.full(B, 0.8, np.float32), noise


def make_sort_inputs(rows=128, n=65536, seed=1, tie_frac=0.01):
    rng = np.random.Generator(np.random.Philox(seed))
    keys = rng.standard_normal((rows, n), dtype=np.float32)
    m = int(n * tie_frac)
    for r in range(rows):
        dst = rng.choice(n, size=m, replace=False)
        src = rng.integers(0, n, size=m)
        keys[r, dst] = keys[r, src]
    payload = np.broadcast_to(np.arange(n, dtype=np.int32), (rows, n)).copy()
    return keys, payload
