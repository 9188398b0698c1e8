"""GPU parity: key/payload sort against the oracle (the stable order is unique, so all variants are bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200 import tax, tumpy
from tests.conftest import exact_match, to_dev, to_np

pytestmark = pytest.mark.gpu

VARIANTS = ["standard", "return_argsort", "return_argsort_stable", "descending", "descending_argsort",
            "descending_stable"]


def _check(cuda, operands, num_keys, variant):
    kw = dict(return_argsort="return_argsort" in variant or "argsort" in variant, is_stable="stable" in variant,
              descending="descending" in variant)
    got = tax.sort([to_dev(x, cuda) for x in operands], num_keys=num_keys, **kw)
    exp = o.sort(operands, num_keys, **kw)
    assert len(got) == len(exp)
    for g, e in zip(got, exp):
        assert exact_match(to_np(g), e)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("size", [128, 256, 2048, 131072])
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("num_arrays,num_keys", [(1, 1), (2, 1), (2, 2)])
def test_sort_comprehensive(cuda, dtype, size, variant, num_arrays, num_keys):
    rows = 16 if size <= 2048 else 4
    rng = np.random.default_rng(0)
    ops = [rng.standard_normal((rows, size)).astype(np.float32) for _ in range(num_arrays)]
    if dtype == "bf16":
        ops = [x.astype(o.bfloat16) for x in ops]  # many ties: the order among them is what is checked
    _check(cuda, ops, num_keys, variant)


@pytest.mark.parametrize("size", [1, 2, 3, 167, 4097, 5000, 8192, 70001])
@pytest.mark.parametrize("dtype", ["f32", "i32"])
def test_sort_ragged_sizes(cuda, size, dtype):
    rng = np.random.default_rng(size)
    keys = rng.integers(-50, 50, (5, size)).astype(np.int32) if dtype == "i32" else rng.standard_normal(
        (5, size)).astype(np.float32)
    payload = rng.integers(0, 1 << 30, (5, size)).astype(np.int32)
    _check(cuda, [keys, payload], 1, "return_argsort_stable")
    _check(cuda, [keys, payload], 1, "descending_stable")


def test_sort_nan_inf_and_signed_zero(cuda):
    x = np.array([[3.0, np.nan, -0.0, 0.0, -np.inf, np.inf, -1.0, np.nan, 0.0, -0.0, 1e-40, -1e-40] * 3], np.float32)
    idx = np.arange(x.shape[1], dtype=np.int32)[None, :].copy()
    for variant in ("return_argsort_stable", "descending_stable"):
        _check(cuda, [x, idx], 1, variant)


def test_sort_key_payload_configuration(cuda):
    # the benchmark's sort configuration at reduced row count: f32 keys with 1 % in-row duplicates, iota payload
    keys, payload = o.make_sort_inputs(rows=6, n=65536, seed=1)
    gk, gp = tax.sort([to_dev(keys, cuda), to_dev(payload, cuda)], num_keys=1, is_stable=True)
    ek, ep = o.sort([keys, payload], 1, is_stable=True)
    assert exact_match(to_np(gk), ek) and np.array_equal(to_np(gp), ep)


def test_sort_full_size_properties(cuda):
    # full benchmark size: sortedness, permutation and stability, checked on the device
    keys, payload = o.make_sort_inputs(rows=128, n=65536, seed=1)
    dk, dp = to_dev(keys, cuda), to_dev(payload, cuda)
    sk, sp = tax.sort([dk, dp], num_keys=1, is_stable=True)
    assert bool((sk[:, 1:] >= sk[:, :-1]).all())
    assert bool((torch.gather(dk, 1, sp.long()) == sk).all())
    ties = sk[:, 1:] == sk[:, :-1]
    assert bool(((sp[:, 1:] > sp[:, :-1]) | ~ties).all())
    assert bool((torch.sort(sp, dim=1).values == dp).all())
    assert int(ties.sum()) > 0


def test_three_operands_two_keys_with_payload(cuda):
    rng = np.random.default_rng(9)
    a = rng.integers(0, 5, (7, 3000)).astype(np.int32)
    b = rng.standard_normal((7, 3000)).astype(np.float32).astype(o.bfloat16)
    c = rng.integers(0, 1 << 20, (7, 3000)).astype(np.int32)
    _check(cuda, [a, b, c], 2, "return_argsort_stable")
    _check(cuda, [a, b, c], 2, "descending_stable")


def test_tumpy_sort_and_argsort(cuda):
    rng = np.random.default_rng(2)
    a = rng.integers(0, 100, (2, 2, 2, 16)).astype(np.int32)
    assert np.array_equal(to_np(tumpy.sort(to_dev(a, cuda))), np.sort(a, axis=-1, kind="stable"))
    assert np.array_equal(to_np(tumpy.argsort(to_dev(a, cuda))), np.argsort(a, axis=-1, kind="stable"))
    assert np.array_equal(to_np(tumpy.sort(to_dev(a, cuda), descending=True)), -np.sort(-a, axis=-1, kind="stable"))
    v = np.array([3, 1, 2], np.int32)
    assert to_np(tumpy.sort(to_dev(v, cuda))).tolist() == [1, 2, 3]
    assert to_np(tumpy.argsort(to_dev(v, cuda))).tolist() == [1, 2, 0]
    flat = tumpy.sort(to_dev(a, cuda), axis=None)
    assert np.array_equal(to_np(flat), np.sort(a.ravel(), kind="stable"))
    with pytest.raises(ValueError):
        tumpy.sort(to_dev(a, cuda), axis=1)


@pytest.mark.parametrize("size", [1 << 19, (1 << 19) + 12345])
def test_sort_rows_beyond_two_to_the_18(cuda, size):
    # the regime of the reference's HBM-resident merge stages (sort.py:588-758, 860-900): rows that no
    # shared-memory tile holds, sorted by the library's multi-pass path
    rng = np.random.default_rng(7)
    keys = rng.standard_normal((2, size)).astype(np.float32)
    keys[1] = np.round(keys[1] * 4) / 4          # many ties: the stable order among them is checked
    pay = rng.integers(0, 1 << 30, (2, size)).astype(np.int32)
    _check(cuda, [keys, pay], 1, "return_argsort_stable")
    _check(cuda, [keys.astype(o.bfloat16)], 1, "descending_argsort")
