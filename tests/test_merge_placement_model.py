"""The placing rule of the vocab-sharded sampler's merge kernel (csrc/sampler.cu, merge_and_sample_kernel), restated
in Python and checked against a plain sort on tie-heavy blocks: the two one-comparison filters never rule out a
candidate whose place is below K, and own position + sum of searches on the composites' high words (with the
+1 for blocks before the candidate's own) is the place in the merged (value desc, token asc) order."""
import numpy as np


def _place_all(blocks, kpb, K, vals):
    n = blocks * kpb
    hi = np.empty(n, dtype=np.int64)                       # inverted key: ascending inside a sorted block
    for b in range(blocks):
        hi[b * kpb:(b + 1) * kpb] = 1000 - np.sort(vals[b])[::-1]
    comp = hi * 100000 + np.arange(n)                      # composite: (key desc, position asc)
    expect = np.sort(comp)[:K]
    merged = np.full(K, -1, dtype=np.int64)
    for i in range(n):
        b, q = divmod(i, kpb)
        if q >= K:
            continue
        c = comp[i]
        probe = K - 1 - q
        if probe < kpb and any(o != b and comp[o * kpb + probe] < c for o in range(blocks)):
            continue                                       # filter 1: one other block alone fills the places
        d = (K - q + blocks - 2) // (blocks - 1)
        if d - 1 < kpb and all(o == b or comp[o * kpb + d - 1] < c for o in range(blocks)):
            continue                                       # filter 2: the other blocks fill them between them
        place, span = q, min(kpb, K - q)
        for o in range(blocks):
            if place >= K:
                break
            if o != b:
                place += int(np.searchsorted(hi[o * kpb:o * kpb + span], hi[i] + (1 if o < b else 0), side="left"))
        if place < K:
            assert merged[place] == -1
            merged[place] = c
    assert (merged == expect).all()


def test_placing_rule_equals_a_sort_on_tie_heavy_blocks():
    rng = np.random.default_rng(0)
    for _ in range(600):
        blocks, kpb = int(rng.integers(2, 9)), int(rng.integers(1, 20))
        K = int(rng.integers(1, blocks * kpb + 1))
        vals = rng.integers(0, int(rng.integers(2, 40)), (blocks, kpb))
        _place_all(blocks, kpb, K, vals)
