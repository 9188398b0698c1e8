"""Two-GPU run of the vocab-sharded sampler, over NCCL and over the peer-memory exchange (skipped with fewer
than two GPUs)."""
import datetime
import os
import queue
import socket

import numpy as np
import pytest

from oracle import tallax_oracle as o

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from tallax_b200 import sampling
        from tests.conftest import to_dev

        B, V = 64, 151936
        x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=4, dtype="bf16")
        vl = V // world
        md = sampling.SamplingMetadata(top_k=to_dev(tk, dev), top_p=to_dev(tp, dev), temperature=to_dev(T, dev))
        tok = sampling.sample_vocab_sharded(None, to_dev(x[:, rank * vl:(rank + 1) * vl], dev), md,
                                            noise_shard=to_dev(noise[:, rank * vl:(rank + 1) * vl], dev), k_cand=50)
        torch.cuda.synchronize()
        # the same steps with the candidates exchanged by the kernels themselves: three steps (both sets of
        # the exchange buffer and a reuse), each must give the tokens of the NCCL path
        ex = sampling.make_vocab_exchange(B, 50, device=dev)
        same = True
        for _ in range(3):
            tok2 = sampling.sample_vocab_sharded(None, to_dev(x[:, rank * vl:(rank + 1) * vl], dev), md,
                                                 noise_shard=to_dev(noise[:, rank * vl:(rank + 1) * vl], dev),
                                                 k_cand=50, exchange=ex)
            same = same and bool((tok2 == tok).all())
        steps, err = ex.state()
        dist.barrier()          # no rank unmaps a buffer that another may still write
        ex.close()
        q.put((rank, tok.cpu().numpy().tolist(), same, steps, err))
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_two_gpus(cuda):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        got = {}
        for _ in range(world):
            try:
                rank, toks, same, steps, err = q.get(timeout=300)
                assert same and steps == 3 and err == 0, (rank, same, steps, err)
            except queue.Empty:
                pytest.fail("a rank delivered no result: exit codes %r" % [p.exitcode for p in procs])
            got[rank] = toks
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        # a rank that is still alive here is stuck (or its peer died): do not leave it behind
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()
    B, V = 64, 151936
    x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=4, dtype="bf16")
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    for r in range(world):
        bad = (np.array(got[r]) != exp) & ~flags
        assert not bad.any()
    assert got[0] == got[1]
