"""The bound of the two-pass top-k kernel (csrc/topk.cu, topk_short_kernel), restated in NumPy: per group the
greatest non-NaN element (a group without one contributes -inf), the K-th largest of the groups' top 16 key
bits as the bound, every element whose top 16 key bits reach it as a candidate.  Whatever the grouping, the
candidates contain the row's top K by (key desc, index asc); NaNs carry the greatest key and pass."""
import numpy as np

from oracle import tallax_oracle as o


def _candidates(row, groups, K):
    n = row.shape[0]
    key16 = (o.sortable_key_u32(row) >> 16).astype(np.int64)
    member = np.arange(n) % groups                       # any assignment of elements to groups will do
    ninf16 = int(o.sortable_key_u32(np.array([-np.inf], np.float32))[0] >> 16)
    maxima = np.full(groups, ninf16, dtype=np.int64)
    ok = ~np.isnan(row)
    np.maximum.at(maxima, member[ok], key16[ok])
    bound = np.sort(maxima)[::-1][K - 1]
    return np.nonzero(key16 >= bound)[0]


def test_candidates_contain_the_top_k():
    rng = np.random.default_rng(1)
    for trial in range(300):
        n = int(rng.integers(8, 3000))
        groups = int(rng.choice([4, 64, 512, 1024]))
        K = int(rng.integers(1, min(n, groups, 128) + 1))
        row = rng.standard_normal(n).astype(np.float32)
        kind = trial % 6
        if kind == 1:
            row = np.round(row * 2) / 2                                  # ties
        elif kind == 2:
            row[rng.random(n) < 0.2] = np.nan
        elif kind == 3:
            row[rng.random(n) < 0.9] = -np.inf
        elif kind == 4:
            row = np.sort(row)                                           # ascending
        elif kind == 5:
            row[::3] = 0.0
            row[1::3] = -0.0
        cand = set(_candidates(row, groups, K).tolist())
        key = o.sortable_key_u32(row).astype(np.int64)
        top = np.lexsort((np.arange(n), -key))[:K]
        assert set(top.tolist()) <= cand, (trial, n, groups, K)
