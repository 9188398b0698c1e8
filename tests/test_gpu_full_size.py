"""Full benchmark sizes, checked on the device through size-independent properties.

The oracle needs minutes at these sizes, so the checks are properties that hold whatever the
size: top-k values against a library top-k (values are unique up to ties, and tie order is
checked by index), gather against a library gather, and "sharded == unsharded" for the sampler.
torch is the checker here, never the thing under test.
"""
import numpy as np
import pytest
import torch

from oracle import tallax_oracle as o
from tallax_b200 import sampling, tax, tumpy
from tallax_b200._src import ops

pytestmark = pytest.mark.gpu


def test_top_k_and_gather_configuration_4(cuda):
    rows, n, k = 1024, 262144, 128
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    x = torch.randn((rows, n), generator=g, device=cuda)
    ref = torch.topk(x, k, dim=1, largest=True, sorted=True)
    vals, idx = tax.top_k(x, k)                       # exact
    assert torch.equal(vals, ref.values)
    assert torch.equal(torch.gather(x, 1, idx.long()), vals)
    same_val = vals[:, 1:] == vals[:, :-1]
    assert bool((idx[:, 1:][same_val] > idx[:, :-1][same_val]).all())   # ties: lower index first
    # single-pass ("approximate") mode: recall against the exact result
    out = ops.top_k(x, k, single_pass=True)
    a_idx = out[1]
    hit = (a_idx.unsqueeze(2) == idx.unsqueeze(1)).any(dim=2).float().mean().item()
    assert hit >= 0.95
    # gather of configuration 4b on the same matrix
    ind = torch.randint(0, n, (rows, 4096), generator=g, device=cuda, dtype=torch.int32)
    got = tumpy.take_along_axis(x, ind, axis=1)
    assert torch.equal(got, torch.gather(x, 1, ind.long()))


def test_vocab_sharded_equals_unsharded_configuration_5(cuda):
    rows, vocab, shards, k = 1024, 151936, 8, 50
    g = torch.Generator(device=cuda)
    g.manual_seed(4)
    x = torch.randn((rows, vocab), generator=g, device=cuda) * 2.0
    rank = torch.rand((rows, vocab), generator=g, device=cuda).argsort(dim=1).argsort(dim=1).float() + 1.0
    x = (x + 4.0 * rank.pow(-1.1)).to(torch.bfloat16)
    del rank
    noise = torch.rand((rows, vocab), generator=g, device=cuda)
    md = sampling.SamplingMetadata(top_k=torch.full((rows,), k, dtype=torch.int32, device=cuda),
                                   top_p=torch.full((rows,), 0.95, device=cuda),
                                   temperature=torch.full((rows,), 0.8, device=cuda))
    whole = sampling.sample(None, x, md, noise=noise)
    vl = vocab // shards
    blocks = [ops.shard_candidates(x[:, s * vl:(s + 1) * vl].contiguous(), s * vl, k,
                                   noise_shard=noise[:, s * vl:(s + 1) * vl].contiguous()) for s in range(shards)]
    merged = ops.merge_and_sample(torch.stack(blocks), md.top_k, md.top_p, md.temperature)
    # The two paths take the softmax over the same top-k set in different summation orders, so a row
    # whose cumulative mass sits within rounding of top_p may differ; everything else is identical.
    differing = torch.nonzero(whole != merged).flatten().tolist()
    assert len(differing) <= 2
    if differing:
        # every such row must be one the oracle flags: cumulative mass within 1e-6 of top_p
        from tests.conftest import to_np
        n = len(differing)
        _, flags = o.sample(to_np(x[differing]), np.full(n, k, np.int32), np.full(n, 0.95, np.float32),
                            np.full(n, 0.8, np.float32), noise=to_np(noise[differing]), return_flags=True)
        assert flags.all(), (differing, flags)
    assert int(whole.min()) >= 0 and int(whole.max()) < vocab
