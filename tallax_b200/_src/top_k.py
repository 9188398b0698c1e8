"""Row-wise top-k (mirror of tallax/_src/top_k.py:385-567)."""
from __future__ import annotations

from tallax_b200 import _lib
from tallax_b200._src import ops

NUM_LANES = 128


def top_dynamic_k(logits, k, max_k: int, block_token: int = 8, num_bins: int = NUM_LANES, bins_topm_unroll: int = 32,
                  bins_topm_schedule=None, guarantee_convergence: bool = False, replace_val=None,
                  interpret: bool = False):
    """Top-`max_k` of every row with a per-row `k` (scalar or [num_tokens]).

    Values descending, ties broken by lower index.  With `replace_val`, positions
    >= k[row] hold it (top_k.py:365-369).  guarantee_convergence=False is the
    single-pass form: returns (vals, idxs, valid, depths, cutoff_vals) where `valid`
    tells whether every row was answered exactly (top_k.py:512-514).
    `num_bins`, `bins_topm_*` and `interpret` are TPU tuning knobs, accepted and ignored.
    max_k may be up to 2048 here (the reference stops at 128).
    """
    num_tokens, vocab = logits.shape
    if num_tokens % block_token != 0:
        raise ValueError("num_tokens must be divisible by block_token")
    if max_k > _lib.TOPK_MAX_K:
        raise NotImplementedError
    if guarantee_convergence:
        return ops.top_k(logits, max_k, k_per_row=k, replace_val=replace_val)
    vals, idxs, valid, depths, cutoff = ops.top_k(logits, max_k, k_per_row=k, replace_val=replace_val,
                                                  single_pass=True)
    return vals, idxs, valid.bool().squeeze(), depths, cutoff


def top_k(logits, k: int, block_token: int = 8, num_bins: int = NUM_LANES, bins_topm_unroll: int = 32,
          bins_topm_schedule=None, interpret: bool = False):
    """Exact top-k with uniform k (top_k.py:527-567): (vals [N, k], idxs [N, k] int32)."""
    return top_dynamic_k(logits, k=k, max_k=k, block_token=block_token, num_bins=num_bins,
                         bins_topm_unroll=bins_topm_unroll, bins_topm_schedule=bins_topm_schedule,
                         guarantee_convergence=True, interpret=interpret)
