"""GPU parity: exact / single-pass / multi-operand top-k against the oracle, bit-exact with ties to the lower index."""
import numpy as np
import pytest

from oracle import tallax_oracle as o
from tallax_b200 import tax
from tallax_b200._src.bitonic_top_k import bitonic_top_k
from tests.conftest import exact_match, to_dev, to_np

pytestmark = pytest.mark.gpu


def _check_topk(cuda, x, k):
    v, i = tax.top_k(to_dev(x, cuda), k, block_token=1)
    ev, ei = o.top_k(x, k)
    assert np.array_equal(to_np(i), ei)
    assert exact_match(to_np(v), ev)


@pytest.mark.parametrize("shape", [(8, 128), (16, 256), (13, 167), (256, 256), (173, 195)])
@pytest.mark.parametrize("dtype", ["f32", "i32"])
def test_bitonic_topk_shapes(cuda, shape, dtype):
    rng = np.random.default_rng(0)
    arr = rng.standard_normal(shape).astype(np.float32) if dtype == "f32" else rng.integers(0, 1000, shape).astype(
        np.int32)
    idx = np.broadcast_to(np.arange(shape[1], dtype=np.int32), shape).copy()
    k = min(128, shape[1])
    v, i = bitonic_top_k([to_dev(arr, cuda), to_dev(idx, cuda)], k=k, num_keys=1, descending=True)
    ev, ei = o.bitonic_top_k([arr, idx], k=k, num_keys=1)
    assert exact_match(to_np(v), ev) and np.array_equal(to_np(i), ei)


def test_topk_config_f32(cuda):
    # benchmark configuration 1: f32 [8, 32768], k=64
    x = np.random.Generator(np.random.Philox(0)).standard_normal((8, 32768), dtype=np.float32)
    _check_topk(cuda, x, 64)


def test_topk_bf16_wide(cuda):
    # the reference's own top-k test shape: bf16 [16, 201088], k=64
    x = np.random.default_rng(0).standard_normal((16, 201088)).astype(np.float32).astype(o.bfloat16)
    _check_topk(cuda, x, 64)


@pytest.mark.parametrize("k", [1, 7, 128, 129, 1000, 2048])
@pytest.mark.parametrize("n", [2048, 50000])
def test_topk_k_range(cuda, k, n):
    x = np.random.default_rng(k).standard_normal((5, n)).astype(np.float32)
    _check_topk(cuda, x, k)


@pytest.mark.parametrize("kind", ["ascending", "descending", "constant", "two_values", "int_ties", "neg_inf_masked",
                                  "nan_and_zero"])
def test_topk_adversarial_rows(cuda, kind):
    n, k = 40000, 100
    rng = np.random.default_rng(3)
    if kind == "ascending":  # every element beats the running threshold: candidate overflow -> radix fallback
        x = np.tile(np.arange(n, dtype=np.float32), (3, 1))
    elif kind == "descending":
        x = np.tile(np.arange(n, 0, -1).astype(np.float32), (3, 1))
    elif kind == "constant":  # one huge tie group: the k lowest indices win
        x = np.full((3, n), 1.5, np.float32)
    elif kind == "two_values":
        x = rng.integers(0, 2, (3, n)).astype(np.float32)
    elif kind == "int_ties":
        x = rng.integers(0, 1000, (3, n)).astype(np.int32)
    elif kind == "neg_inf_masked":  # logits with most of the vocabulary masked out
        x = rng.standard_normal((3, n)).astype(np.float32)
        x[:, rng.random(n) < 0.999] = -np.inf
    else:
        x = rng.standard_normal((3, n)).astype(np.float32)
        x[:, ::7] = 0.0
        x[:, 3::7] = -0.0
        x[0, 5] = np.nan
    _check_topk(cuda, x, k)


def test_top_dynamic_k_masks_with_replace_val(cuda):
    x = np.random.default_rng(1).standard_normal((16, 30000)).astype(np.float32)
    k = np.random.default_rng(2).integers(1, 129, 16).astype(np.int32)
    v, i = tax.top_dynamic_k(to_dev(x, cuda), to_dev(k, cuda), max_k=128, guarantee_convergence=True,
                             replace_val=-1e12)
    ev, ei = o.top_dynamic_k(x, k, 128, replace_val=-1e12)
    assert np.array_equal(to_np(v), ev) and np.array_equal(to_np(i), ei)


def test_single_pass_topk_contract(cuda):
    # guarantee_convergence=False: five outputs; iid rows are answered exactly (valid), recall 1.0
    x = np.random.Generator(np.random.Philox(3)).standard_normal((64, 262144), dtype=np.float32)
    v, i, valid, depths, cutoff = tax.top_dynamic_k(to_dev(x, cuda), 128, max_k=128, guarantee_convergence=False)
    ev, ei = o.top_k(x, 128)
    assert bool(valid)
    assert o.topk_recall(to_np(i), ei) >= 0.95
    assert np.array_equal(to_np(i), ei) and np.array_equal(to_np(v), ev)
    assert depths.shape == (64,) and cutoff.shape == (64,)
    assert np.all(to_np(cutoff) <= ev[:, -1])  # the reported pivot is a lower bound of the k-th value
    # an ascending row defeats the single pass: valid is cleared, the answer is still k in-range distinct indices
    bad = np.tile(np.arange(100000, dtype=np.float32), (8, 1))
    v, i, valid, _, _ = tax.top_dynamic_k(to_dev(bad, cuda), 64, max_k=64, guarantee_convergence=False)
    assert not bool(valid)
    ii = to_np(i)
    assert ii.min() >= 0 and ii.max() < 100000 and all(len(set(r.tolist())) == 64 for r in ii)


@pytest.mark.parametrize("rows,n,k,dtype", [(8, 32768, 64, "f32"), (3, 65536, 256, "f32"), (16, 32768, 128, "bf16"),
                                             (1, 131072, 17, "f32"), (5, 49152, 50, "i32")])
def test_topk_of_a_few_long_rows_split_over_ctas(cuda, rows, n, k, dtype):
    # the rows are cut into parts whose candidates a second pass merges; ties across and inside parts must
    # still come out with the lower index first
    from tallax_b200 import _lib
    assert _lib.load().tlx_top_k_workspace_bytes(rows, n, k) > 0       # this shape does take the split path
    rng = np.random.default_rng(rows * 1000 + k)
    if dtype == "i32":
        x = rng.integers(-50, 51, (rows, n)).astype(np.int32)
    else:
        x = np.round(rng.standard_normal((rows, n)).astype(np.float32) * 8) / 8      # eighths: plenty of ties
        x[0, ::4096] = 7.0                                                           # a tie group across all parts
        if rows > 1:
            x[1] = -3.0                                                              # one value only
        if dtype == "bf16":
            x = x.astype(o.bfloat16)
    _check_topk(cuda, x, k)
    if dtype == "f32":
        kk = rng.integers(1, k + 1, rows).astype(np.int32)
        v, i = tax.top_dynamic_k(to_dev(x, cuda), to_dev(kk, cuda), max_k=k, replace_val=-1e12, block_token=1,
                                 guarantee_convergence=True)
        ev, ei = o.top_dynamic_k(x, kk, k, replace_val=-1e12)
        assert exact_match(to_np(v), ev) and np.array_equal(to_np(i), ei)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("n,k", [(2048, 128), (18992, 50), (40001, 7), (70000, 128)])
def test_topk_of_many_rows_two_pass_kernel(cuda, dtype, n, k):
    # 256 rows and more with k <= 128 take the two-pass kernel (bound from group maxima); rows over 128 KB
    # take the bound from a sample of the row.  One row each of the shapes that stress it: ascending and
    # descending (the sampled bound is far too low or exact), one value only and two values (candidate
    # overflow -> exact fallback), eighths (ties around the bound), NaNs, infinities, signed zeros, a row
    # whose large values all sit in the part the sample skips.
    rows = 260
    rng = np.random.default_rng(n + k)
    x = rng.standard_normal((rows, n)).astype(np.float32) * 2
    x[0] = np.arange(n, dtype=np.float32) / 64
    x[1] = np.arange(n, 0, -1).astype(np.float32) / 64
    x[2] = 1.5
    x[3] = rng.integers(0, 2, n).astype(np.float32)
    x[4] = np.round(x[4] * 8) / 8
    x[5, rng.random(n) < 0.01] = np.nan
    x[6, rng.random(n) < 0.999] = -np.inf
    x[7, ::5] = np.inf
    x[8, ::7] = 0.0
    x[8, 3::7] = -0.0
    x[8] = np.minimum(x[8], 0.0)
    x[9] = -np.abs(x[9])
    x[9, 128:256] = 50.0 + np.arange(128, dtype=np.float32)      # only in the 2 KB pieces a sampled pass skips
    x[10] = -np.inf
    x[10, :k - 1] = 1.0                                            # fewer finite values than k
    if dtype == "bf16":
        x = x.astype(o.bfloat16)
    elif dtype == "f16":
        x = x.astype(np.float16)
    _check_topk(cuda, x, k)


def test_topk_two_pass_kernel_with_unaligned_rows(cuda):
    # a row stride that is not a multiple of 16 bytes: the traversal's scalar head and tail
    import torch
    rng = np.random.default_rng(5)
    base = rng.standard_normal((300, 5003)).astype(np.float32).astype(o.bfloat16)
    xd = to_dev(base, cuda)[:, 1:5002]
    v, i = tax.top_k(xd, 33, block_token=1)
    ev, ei = o.top_k(np.ascontiguousarray(base[:, 1:5002]), 33)
    assert np.array_equal(to_np(i), ei) and exact_match(to_np(v), ev)


_FORCED_CHILD = r"""
import sys
sys.path.insert(0, %r)
import numpy as np, torch
from oracle import tallax_oracle as o
from tallax_b200 import tax
from tests.conftest import exact_match, to_dev, to_np
dev = torch.device("cuda", 0)
rng = np.random.default_rng(11)
for dtype in ("bf16", "f16", "f32"):
    for rows, n, k in [(5, 520, 50), (7, 100, 100), (3, 8, 8), (9, 2060, 128), (4, 1031, 17), (2, 33000, 64)]:
        x = rng.standard_normal((rows, n)).astype(np.float32)
        x[0, k - 1:] = -np.inf                 # fewer finite values than k: the bound is the bin of -inf
        if rows > 1:
            x[1] = np.round(x[1] * 4) / 4      # ties
        if rows > 2:
            x[2, ::3] = np.nan
        x = x.astype(o.bfloat16) if dtype == "bf16" else x.astype(np.float16) if dtype == "f16" else x
        v, i = tax.top_k(to_dev(x, dev), k, block_token=1)
        ev, ei = o.top_k(x, k)
        assert np.array_equal(to_np(i), ei), (dtype, rows, n, k)
        assert exact_match(to_np(v), ev), (dtype, rows, n, k)
print("ok")
"""


def test_two_pass_kernel_forced_on_small_and_odd_shapes(cuda):
    # TLX_TOPK_PATH=short (read once per process, hence the child) sends every eligible call through the
    # two-pass kernel, also shapes the heuristic would keep away from it: rows shorter than a vector, vector
    # counts that are no multiple of eight (padding of the per-vector maxima), a bound in the bin of -inf
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TLX_TOPK_PATH="short")
    res = subprocess.run([sys.executable, "-c", _FORCED_CHILD % root], capture_output=True, text=True, env=env,
                         timeout=600)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
