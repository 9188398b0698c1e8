"""GPU: the *_dev entry points (PRNG key and batch offset as device operands) give the results of the
host-operand entry points, and follow a key that changes on the device between replays of a CUDA graph."""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200._src import ops
from tests.conftest import to_dev, to_np

pytestmark = pytest.mark.gpu

KEY = (0x1234ABCD, 0x0F1E2D3C)


def _key_dev(cuda, key=KEY):
    return torch.tensor(key, dtype=torch.int64, device=cuda).to(torch.int32)


@pytest.mark.parametrize("dtype,V", [("bf16", 128256), ("bf16", 4096), ("f32", 50000)])
def test_sample_with_device_key_and_offset(cuda, dtype, V):
    B, off = 40, 24
    x, tk, tp, T, _ = o.make_sampling_inputs(B=B, V=V, seed=7, dtype=dtype)
    tk = np.minimum(tk, V).astype(np.int32)
    args = [to_dev(a, cuda) for a in (x, tk, tp, T)]
    host = ops.sample(*args, rng_key=KEY, dim0_offset=off).clone()
    dev_key = ops.sample(*args, rng_key=_key_dev(cuda), dim0_offset=off).clone()
    dev_both = ops.sample(*args, rng_key=_key_dev(cuda),
                          dim0_offset=torch.tensor(off, dtype=torch.int32, device=cuda)).clone()
    dev_off = ops.sample(*args, rng_key=KEY, dim0_offset=torch.tensor(off, dtype=torch.int32, device=cuda)).clone()
    assert torch.equal(host, dev_key) and torch.equal(host, dev_both) and torch.equal(host, dev_off)
    # and against the oracle's threefry noise
    exp, flags = o.sample(x, tk, tp, T, rng_key=KEY, dim0_offset=off, return_flags=True)
    assert not ((to_np(host) != exp) & ~flags).any()


def test_sample_with_dense_noise_and_device_offset(cuda):
    B, V, off = 16, 128256, 8
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B + off, V=V, seed=9, dtype="bf16")
    args = [to_dev(a[off:] if a.shape[0] == B + off else a, cuda) for a in (x, tk, tp, T)]
    dn = to_dev(noise, cuda)
    host = ops.sample(*args, noise=dn, dim0_offset=off).clone()
    dev = ops.sample(*args, noise=dn, dim0_offset=torch.tensor(off, dtype=torch.int32, device=cuda)).clone()
    assert torch.equal(host, dev)
    exp, flags = o.sample(x[off:], tk[off:], tp[off:], T[off:], noise=noise[off:], return_flags=True)
    assert not ((to_np(dev) != exp) & ~flags).any()


def test_device_key_is_read_when_the_graph_runs(cuda):
    B, V = 32, 128256
    x, tk, tp, T, _ = o.make_sampling_inputs(B=B, V=V, seed=3, dtype="bf16")
    args = [to_dev(a, cuda) for a in (x, tk, tp, T)]
    ws = ops.SampleWorkspace(B, V, cuda)
    key = _key_dev(cuda)
    ops.sample(*args, rng_key=key, workspace=ws)   # warm-up outside the capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            ops.sample(*args, rng_key=key, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    for new_key in ((1, 2), (0xDEADBEEF, 0x9E3779B9)):
        key.copy_(_key_dev(cuda, new_key))
        g.replay()
        torch.cuda.synchronize()
        got = ws.tokens.clone()
        want = ops.sample(*args, rng_key=new_key).clone()
        assert torch.equal(got, want)


def test_candidate_sampler_noise_and_shard_candidates_with_device_operands(cuda):
    rng = np.random.default_rng(5)
    B, k, V, off = 24, 64, 32000, 16
    vals = -np.sort(-rng.standard_normal((B, k)).astype(np.float32) * 3, axis=1)
    idx = np.stack([rng.choice(V, k, replace=False) for _ in range(B)]).astype(np.int32)
    tp = rng.uniform(0.5, 1.0, B).astype(np.float32)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    a = [to_dev(v, cuda) for v in (vals, idx, tp, T)]
    off_dev = torch.tensor(off, dtype=torch.int32, device=cuda)
    host = ops.top_p_and_sample(*a, vocab_size=V, replace_val=-1e12, rng_key=KEY, dim0_offset=off)
    dev = ops.top_p_and_sample(*a, vocab_size=V, replace_val=-1e12, rng_key=_key_dev(cuda), dim0_offset=off_dev)
    assert torch.equal(host, dev)
    # counter-based noise and the Gumbel arg-max with indexed noise
    i0 = to_dev(rng.integers(0, 100, (8, 256)).astype(np.int32), cuda)
    i1 = to_dev(rng.integers(0, V, (8, 256)).astype(np.int32), cuda)
    assert torch.equal(ops.sparse_random_uniform(KEY, i0, i1, V), ops.sparse_random_uniform(_key_dev(cuda), i0, i1, V))
    lg = to_dev(rng.standard_normal((8, 256)).astype(np.float32), cuda)
    h = ops.gumbel_argmax(KEY, lg, i0, i1, V, 1)
    d = ops.gumbel_argmax(_key_dev(cuda), lg, i0, i1, V, 1)
    assert all(torch.equal(x, y) for x, y in zip(h, d))
    # one vocab shard's candidates with key noise
    xs, _, _, _, _ = o.make_sharded_inputs(B=16, V=32768, seed=8, dtype="bf16")
    dx = to_dev(xs[:, 8192:16384].copy(), cuda)
    h = ops.shard_candidates(dx, 8192, 50, rng_key=KEY, vocab_total=32768, dim0_offset=off)
    d = ops.shard_candidates(dx, 8192, 50, rng_key=_key_dev(cuda), vocab_total=32768, dim0_offset=off_dev)
    assert torch.equal(h, d)
