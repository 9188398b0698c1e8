"""CPU tests of the vLLM-convention front end (tallax_b200/vllm_adapter.py): the parameter mapping, the min_p
value test, per-request seeds.  The CUDA sampler is replaced by the oracle; what is checked is the host logic."""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200 import vllm_adapter as va


def _oracle_sample(key, logits, md):
    x = logits.numpy() if logits.dtype != torch.bfloat16 else logits.float().numpy()
    return torch.from_numpy(o.sample(x, md.top_k.numpy(), md.top_p.numpy(), md.temperature.numpy(), rng_key=tuple(key)))


def _row_max(x):
    return x.max(dim=1).values


def test_top_k_conventions():
    got = va.normalize_top_k([-1, 0, 1, 50, 999, 1000, 5000], 7, 1000)
    assert got.dtype == torch.int32 and got.tolist() == [0, 0, 1, 50, 999, 0, 0]
    assert va.normalize_top_k(None, 3, 10).tolist() == [0, 0, 0]
    assert va.normalize_top_k(-1, 3, 10).tolist() == [0, 0, 0]
    with pytest.raises(ValueError):
        va.normalize_top_k([-2], 1, 10)
    with pytest.raises(ValueError):
        va.normalize_top_k([1, 2], 3, 10)


def test_min_p_threshold_is_the_probability_test():
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((6, 500)).astype(np.float32) * 3)
    T = torch.tensor([0.5, 1.0, 1.5, 0.7, 1.0, 0.0])
    min_p = torch.tensor([0.05, 0.2, 0.01, 0.0, 1.0, 0.3])
    thr = va.min_p_threshold(x.max(dim=1).values, T, min_p)
    for b in range(5):
        p = torch.softmax(x[b].double() / float(T[b]), dim=0)
        keep_prob = p >= float(min_p[b]) * p.max()
        keep_val = x[b] >= thr[b]
        # identical except elements whose probability ratio is within rounding of min_p
        ratio = (p / p.max() - float(min_p[b])).abs()
        assert bool(((keep_prob == keep_val) | (ratio < 1e-6)).all())
    assert thr[3] == -np.inf and thr[5] == -np.inf     # min_p = 0 and a greedy row cut nothing
    assert bool((x[4] >= thr[4]).sum() == 1)            # min_p = 1 keeps the maximum only


def test_sample_maps_parameters_and_matches_the_oracle_on_cpu():
    rng = np.random.default_rng(1)
    B, V = 10, 400
    x = torch.from_numpy(rng.standard_normal((B, V)).astype(np.float32) * 3)
    params = va.VllmSamplingParams(temperature=[0.0, 1.0, 0.7, 1.3, 1.0, 1.0, 0.9, 1.0, 1.0, 1.0],
                                   top_k=[-1, 0, 5, 50, V, V + 7, 1, 20, -1, 3],
                                   top_p=[1.0, 0.9, 1.0, 0.5, 0.95, 1.0, 1.0, 0.8, 0.7, 1.0])
    key = (11, 22)
    got = va.sample(key, x, params, sample_fn=_oracle_sample, row_max_fn=_row_max)
    tk = np.array([0, 0, 5, 50, 0, 0, 1, 20, 0, 3], np.int32)
    exp = o.sample(x.numpy(), tk, np.array(params.top_p, np.float32), np.array(params.temperature, np.float32),
                   rng_key=key)
    assert got.dtype == torch.int32 and np.array_equal(got.numpy(), exp)
    assert got[0] == int(x[0].argmax()) and got[6] == int(x[6].argmax())   # temperature 0 and top_k 1 are greedy


def test_min_p_rows_are_filtered_and_others_untouched():
    rng = np.random.default_rng(2)
    B, V = 6, 300
    x = torch.from_numpy(rng.standard_normal((B, V)).astype(np.float32) * 2)
    seen = {}

    def spy(key, logits, md):
        seen["x"] = logits.clone()
        return _oracle_sample(key, logits, md)

    params = va.VllmSamplingParams(temperature=1.0, min_p=[0.0, 0.5, 0.0, 1.0, 0.1, 0.0])
    tok = va.sample((3, 4), x, params, sample_fn=spy, row_max_fn=_row_max)
    xs = seen["x"]
    assert torch.equal(xs[0], x[0]) and torch.equal(xs[2], x[2]) and torch.equal(xs[5], x[5])
    assert int(torch.isfinite(xs[3]).sum()) == 1 and tok[3] == int(x[3].argmax())
    p = torch.softmax(x[1].double(), 0)
    assert torch.equal(torch.isfinite(xs[1]), p >= 0.5 * p.max())
    assert torch.equal(x, x.clone()) and not torch.equal(xs, x)     # the caller's logits are not modified


def test_seeded_requests_do_not_depend_on_their_place_in_the_batch():
    rng = np.random.default_rng(3)
    V = 200
    rows = torch.from_numpy(rng.standard_normal((5, V)).astype(np.float32) * 2)
    seeds = [None, 1234, None, 99, None]
    a = va.sample((7, 8), rows, va.VllmSamplingParams(top_k=20, seeds=seeds), step=3, sample_fn=_oracle_sample,
                  row_max_fn=_row_max)
    perm = [3, 0, 1, 4, 2]
    b = va.sample((70, 80), rows[perm], va.VllmSamplingParams(top_k=20, seeds=[seeds[i] for i in perm]), step=3,
                  sample_fn=_oracle_sample, row_max_fn=_row_max)
    assert a[1] == b[perm.index(1)] and a[3] == b[perm.index(3)]      # same seed, same step -> same token
    c = va.sample((7, 8), rows, va.VllmSamplingParams(top_k=20, seeds=seeds), step=4, sample_fn=_oracle_sample,
                  row_max_fn=_row_max)
    assert va.request_key(1234, 3) != va.request_key(1234, 4) and va.request_key(1, 0) != va.request_key(2, 0)
    assert c.shape == a.shape


def test_scale_before_top_p_gives_vllms_order():
    rng = np.random.default_rng(4)
    B, V = 4, 300
    x = torch.from_numpy(rng.standard_normal((B, V)).astype(np.float32) * 3)
    T = np.array([0.5, 2.0, 1.0, 0.0], np.float32)
    params = va.VllmSamplingParams(temperature=T, top_p=[0.8, 0.8, 0.8, 0.8], top_k=-1)
    got = va.sample((5, 6), x, params, scale_before_top_p=True, sample_fn=_oracle_sample, row_max_fn=_row_max)
    scaled = x.numpy() / np.where(T > 0, T, 1.0)[:, None]
    exp = o.sample(scaled.astype(np.float32), np.zeros(B, np.int32), np.full(B, 0.8, np.float32),
                   np.where(T > 0, 1.0, 0.0).astype(np.float32), rng_key=(5, 6))
    assert np.array_equal(got.numpy(), exp)


def test_argument_errors():
    x = torch.zeros((2, 10))
    for bad in (va.VllmSamplingParams(top_p=[0.0, 1.0]), va.VllmSamplingParams(temperature=[-1.0, 1.0]),
                va.VllmSamplingParams(min_p=[2.0, 0.0]), va.VllmSamplingParams(seeds=[1])):
        with pytest.raises(ValueError):
            va.sample((0, 0), x, bad, sample_fn=_oracle_sample, row_max_fn=_row_max)
    with pytest.raises(ValueError):
        va.sample((0, 0), torch.zeros(10), va.VllmSamplingParams(), sample_fn=_oracle_sample, row_max_fn=_row_max)


@pytest.mark.gpu
def test_adapter_on_the_gpu_matches_the_cpu_stand_ins(cuda):
    rng = np.random.default_rng(5)
    B, V = 12, 32768
    xh = torch.from_numpy(rng.standard_normal((B, V)).astype(np.float32) * 3)
    seeds = [None] * B
    seeds[2], seeds[7] = 42, 4242
    params = va.VllmSamplingParams(temperature=[0.0, 1.0, 0.7, 1.3, 1.0, 1.0, 0.9, 1.0, 1.0, 1.0, 0.8, 1.1],
                                   top_k=[-1, 0, 5, 50, V, 1, 1, 20, -1, 3, 100, 1000],
                                   top_p=[1.0, 0.9, 1.0, 0.5, 0.95, 1.0, 1.0, 0.8, 0.7, 1.0, 0.9, 0.99],
                                   min_p=[0, 0, 0.1, 0, 0, 0, 0, 0.3, 0.02, 0, 0, 0], seeds=seeds)
    want = va.sample((9, 10), xh, params, step=2, sample_fn=_oracle_sample, row_max_fn=_row_max)
    got = va.sample((9, 10), xh.to(cuda), params, step=2)
    assert torch.equal(got.cpu(), want)
