"""The peer-memory candidate exchange of the vocab-sharded sampler on ONE GPU: the ranks are stood in for by
successive launches on one stream (every rank's candidate kernel, then every rank's merge kernel), so that no
kernel ever waits for one that has not run.  The two-GPU run is in test_gpu_distributed.py."""
import numpy as np
import pytest

from oracle import tallax_oracle as o

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,dtype,k", [(1, "bf16", 50), (2, "bf16", 50), (4, "f32", 64), (8, "bf16", 128)])
def test_exchange_matches_the_gathered_path_and_the_oracle(cuda, world, dtype, k):
    import torch
    from tallax_b200 import sampling
    from tallax_b200._src import ops
    from tests.conftest import to_dev

    dev = torch.device("cuda", 0)
    B, V = 48, 4096 * world
    group = ops.Exchange.local_group(B, k, world, dev)
    try:
        for step in range(3):
            x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=10 + step, dtype=dtype)
            tk = np.minimum(tk, k).astype(np.int32)
            vl = V // world
            xs = [to_dev(x[:, r * vl:(r + 1) * vl], dev).contiguous() for r in range(world)]
            ns = [to_dev(noise[:, r * vl:(r + 1) * vl], dev).contiguous() for r in range(world)]
            dtk, dtp, dT = to_dev(tk, dev), to_dev(tp, dev), to_dev(T, dev)
            for r in range(world):
                ops.exchange_shard_candidates(xs[r], r * vl, group[r], noise_shard=ns[r], vocab_total=V)
            toks = [ops.exchange_merge_and_sample(group[r], dtk, dtp, dT).cpu().numpy() for r in range(world)]
            # the gathered path on the same shards
            gathered = torch.stack([ops.shard_candidates(xs[r], r * vl, k, noise_shard=ns[r], vocab_total=V)
                                    for r in range(world)])
            ref = ops.merge_and_sample(gathered, dtk, dtp, dT).cpu().numpy()
            exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
            for r in range(world):
                assert (toks[r] == ref).all()
                assert not ((toks[r] != exp) & ~flags).any()
                assert group[r].state() == (step + 1, 0)
    finally:
        for e in group:
            e.close()


def test_exchange_with_key_noise(cuda):
    import torch
    from tallax_b200._src import ops
    from tests.conftest import to_dev

    dev = torch.device("cuda", 0)
    world, B, V, k = 2, 16, 8192, 32
    group = ops.Exchange.local_group(B, k, world, dev)
    try:
        x, tk, tp, T, _ = o.make_sharded_inputs(B=B, V=V, seed=3, dtype="bf16")
        tk = np.minimum(tk, k).astype(np.int32)
        vl = V // world
        key = (7, 11)
        xs = [to_dev(x[:, r * vl:(r + 1) * vl], dev).contiguous() for r in range(world)]
        dtk, dtp, dT = to_dev(tk, dev), to_dev(tp, dev), to_dev(T, dev)
        for r in range(world):
            ops.exchange_shard_candidates(xs[r], r * vl, group[r], rng_key=key, vocab_total=V, dim0_offset=5)
        tok = ops.exchange_merge_and_sample(group[0], dtk, dtp, dT).cpu().numpy()
        ops.exchange_merge_and_sample(group[1], dtk, dtp, dT)
        gathered = torch.stack([ops.shard_candidates(xs[r], r * vl, k, rng_key=key, vocab_total=V, dim0_offset=5)
                                for r in range(world)])
        ref = ops.merge_and_sample(gathered, dtk, dtp, dT).cpu().numpy()
        assert (tok == ref).all()
    finally:
        for e in group:
            e.close()


def test_a_missing_rank_is_reported_not_waited_for_forever(cuda):
    """Only rank 0 of two delivers: the merge kernel's bounded wait (two seconds) gives up, sets the status and
    the buffer's error word, and the context stays usable."""
    import torch
    from tallax_b200._src import ops
    from tests.conftest import to_dev

    dev = torch.device("cuda", 0)
    world, B, V, k = 2, 4, 4096, 16
    group = ops.Exchange.local_group(B, k, world, dev)
    try:
        x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=1, dtype="bf16")
        vl = V // world
        ops.exchange_shard_candidates(to_dev(x[:, :vl], dev).contiguous(), 0, group[0],
                                      noise_shard=to_dev(noise[:, :vl], dev).contiguous(), vocab_total=V)
        ops.exchange_merge_and_sample(group[0], to_dev(np.minimum(tk, k).astype(np.int32), dev), to_dev(tp, dev),
                                      to_dev(T, dev))
        torch.cuda.synchronize()
        assert int(group[0].status.item()) == 1
        assert group[0].state()[1] == 1
        assert float(torch.ones(4, device=dev).sum()) == 4.0       # the context still works
    finally:
        for e in group:
            e.close()


def test_exchange_steps_replayed_from_a_cuda_graph(cuda):
    """The set a step uses is the low bit of a counter in the buffer that the merge kernel advances: a captured
    step can be replayed any number of times, interleaved with eager steps, without host bookkeeping."""
    import torch
    from tallax_b200._src import ops
    from tests.conftest import to_dev

    dev = torch.device("cuda", 0)
    B, V, k = 40, 8192, 32
    (ex,) = ops.Exchange.local_group(B, k, 1, dev)
    try:
        inputs = []
        for seed in (21, 22, 23, 24):
            x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=seed, dtype="bf16")
            tk = np.minimum(tk, k).astype(np.int32)
            exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
            inputs.append((to_dev(x, dev), to_dev(noise, dev), exp, flags))
        dtk, dtp, dT = to_dev(tk, dev), to_dev(tp, dev), to_dev(T, dev)
        sx, sn = torch.empty_like(inputs[0][0]), torch.empty_like(inputs[0][1])
        out = torch.empty(B, dtype=torch.int32, device=dev)

        def step():
            ops.exchange_shard_candidates(sx, 0, ex, noise_shard=sn, vocab_total=V)
            ops.exchange_merge_and_sample(ex, dtk, dtp, dT, out=out)

        sx.copy_(inputs[0][0]); sn.copy_(inputs[0][1])
        step()                                   # eager: step 1 (also loads the kernels before the capture)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()                               # captured, not run
        done = 1
        for j, (x, noise, exp, flags) in enumerate(inputs):
            sx.copy_(x); sn.copy_(noise)
            if j == 2:
                step()                           # an eager step between replays
            else:
                graph.replay()
            done += 1
            got = out.cpu().numpy()
            assert not ((got != exp) & ~flags).any(), j
            assert ex.state() == (done, 0)
    finally:
        ex.close()


def test_a_call_with_other_extents_than_the_buffers_touches_nothing(cuda):
    import torch
    from tallax_b200._src import ops
    from tests.conftest import to_dev

    dev = torch.device("cuda", 0)
    B, V = 8, 4096
    (ex,) = ops.Exchange.local_group(B, 16, 1, dev)
    try:
        x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=5, dtype="bf16")
        ex.k_cand = 32                      # the buffer was made for 16 candidates per row
        ops.exchange_shard_candidates(to_dev(x, dev), 0, ex, noise_shard=to_dev(noise, dev), vocab_total=V)
        tok = ops.exchange_merge_and_sample(ex, to_dev(np.minimum(tk, 16).astype(np.int32), dev), to_dev(tp, dev),
                                            to_dev(T, dev))
        torch.cuda.synchronize()
        assert (tok.cpu().numpy() == -1).all()
        assert int(ex.status.item()) == 2
        assert ex.state() == (0, 2)          # no step was made, the mark is in the buffer
    finally:
        ex.close()


@pytest.mark.parametrize("world,k", [(2, 32), (4, 32), (8, 16), (3, 50)])
def test_merge_of_sorted_blocks_with_ties_and_every_top_k(cuda, world, k):
    """The merge places candidates without sorting: values in quarters (equal values across and inside the
    shards' blocks, so the token order decides), top_k from 1 to all candidates and 0 (keep all), rows with a
    temperature of 0.  Checked against the oracle's merge of the very same candidates."""
    import torch
    from tallax_b200._src import ops
    from tests.conftest import to_dev, to_np

    dev = torch.device("cuda", 0)
    B, vl = 96, 1024
    rng = np.random.default_rng(100 * world + k)
    x = (np.round(rng.standard_normal((B, vl * world)).astype(np.float32) * 4) / 4).astype(o.bfloat16)
    noise = rng.random((B, vl * world), dtype=np.float32)
    gathered = torch.stack([ops.shard_candidates(to_dev(np.ascontiguousarray(x[:, r * vl:(r + 1) * vl]), dev), r * vl, k,
                                                 noise_shard=to_dev(np.ascontiguousarray(noise[:, r * vl:(r + 1) * vl]), dev),
                                                 vocab_total=vl * world) for r in range(world)])
    tk = rng.integers(0, world * k + 1, B).astype(np.int32)      # 0 keeps all world * k candidates
    tk[:4] = [1, world * k, k, 0]
    tp = rng.uniform(0.5, 1.0, B).astype(np.float32)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[5] = 0.0
    tok = to_np(ops.merge_and_sample(gathered, to_dev(tk, dev), to_dev(tp, dev), to_dev(T, dev)))
    g = to_np(gathered)
    cv = np.concatenate([g[s, 0] for s in range(world)], axis=1)
    ci = np.concatenate([g[s, 1].view(np.int32) for s in range(world)], axis=1)
    cn = np.concatenate([g[s, 2] for s in range(world)], axis=1)
    exp, flags = o.merge_and_sample(cv, ci, cn, tk, tp, T, return_flags=True)
    assert not ((tok != exp) & ~flags).any()
    assert flags.mean() < 0.2
