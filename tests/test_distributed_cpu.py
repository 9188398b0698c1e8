"""Host-side logic of the multi-rank paths, on CPU ranks over gloo (world size 2).

The CUDA kernels are replaced by their oracle equivalents inside the child processes, so what
is exercised here is the plumbing of `sampling.sample_vocab_sharded`: shard offsets, the packed
[3, rows, k] candidate block, the all-gather layout and the strided view the merge reads; and the
row-offset rule of batch sharding.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tallax_oracle as o


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _install_cpu_kernels():
    """Oracle stand-ins with the C ABI's data layout, for CPU tensors."""
    from tallax_b200._src import ops

    def shard_candidates(logits_shard, col_offset, k_cand, *, noise_shard=None, rng_key=None, vocab_total=None,
                         dim0_offset=0, out=None):
        x = logits_shard.float().numpy()
        vals, idx, u = o.shard_candidates(x, col_offset, k_cand, noise_shard.numpy())
        block = out if out is not None else torch.empty((3,) + vals.shape, dtype=torch.float32)
        block[0] = torch.from_numpy(vals)
        block[1] = torch.from_numpy(idx.view(np.float32))   # token ids travel bit-cast in the f32 block
        block[2] = torch.from_numpy(u)
        return block

    def merge_and_sample(gathered, top_k_, top_p, temperature, out=None):
        n_shards, _, rows, k = gathered.shape
        g = gathered.numpy()
        cv = np.concatenate([g[s, 0] for s in range(n_shards)], axis=1)
        ci = np.concatenate([g[s, 1].view(np.int32) for s in range(n_shards)], axis=1)
        cn = np.concatenate([g[s, 2] for s in range(n_shards)], axis=1)
        tok = torch.from_numpy(o.merge_and_sample(cv, ci, cn, top_k_.numpy(), top_p.numpy(), temperature.numpy()))
        if out is not None:
            out.copy_(tok)
            return out
        return tok

    ops.shard_candidates = shard_candidates
    ops.merge_and_sample = merge_and_sample

    # The peer-memory exchange: the buffers become host objects and a rank's stores into its peers' buffers an
    # all-gather at merge time; what stays under test is make_vocab_exchange (handles gathered in rank order,
    # own entry not opened) and the routing of sample_vocab_sharded(..., exchange=).
    class Exchange:
        def __init__(self, rows, k_cand, world):
            self.rows, self.k_cand, self.world, self.rank, self.block, self.seen = rows, k_cand, world, None, None, None

        @classmethod
        def create(cls, rows, k_cand, world, device=None):
            self = cls(rows, k_cand, world)
            self.handle = b"buffer of rank %d" % dist.get_rank()
            return self

        def attach(self, rank, handles):
            self.rank, self.seen = rank, list(handles)
            return self

    def exchange_shard_candidates(logits_shard, col_offset, exchange, *, noise_shard=None, rng_key=None,
                                  vocab_total=None, dim0_offset=0):
        exchange.block = shard_candidates(logits_shard, col_offset, exchange.k_cand, noise_shard=noise_shard)
        exchange.args = (col_offset, vocab_total)

    def exchange_merge_and_sample(exchange, top_k_, top_p, temperature, out=None):
        gathered = torch.empty((exchange.world,) + tuple(exchange.block.shape), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered.view((exchange.world * 3,) + tuple(exchange.block.shape[1:])), exchange.block)
        return merge_and_sample(gathered, top_k_, top_p, temperature, out=out)

    ops.Exchange = Exchange
    ops.exchange_shard_candidates = exchange_shard_candidates
    ops.exchange_merge_and_sample = exchange_merge_and_sample


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        _install_cpu_kernels()
        from tallax_b200 import sampling

        B, V = 12, 4096
        x, tk, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=4, dtype="f32")
        tk = np.random.default_rng(0).integers(1, 33, B).astype(np.int32)
        vl = V // world
        md = sampling.SamplingMetadata(top_k=torch.from_numpy(tk), top_p=torch.from_numpy(tp),
                                       temperature=torch.from_numpy(T))
        tok = sampling.sample_vocab_sharded(None, torch.from_numpy(x[:, rank * vl:(rank + 1) * vl].copy()), md,
                                            noise_shard=torch.from_numpy(noise[:, rank * vl:(rank + 1) * vl].copy()),
                                            k_cand=32)
        # the same step through the exchange form
        ex = sampling.make_vocab_exchange(B, 32)
        assert ex.rank == rank and ex.seen == [b"buffer of rank 0", b"buffer of rank 1"]
        tok2 = sampling.sample_vocab_sharded(None, torch.from_numpy(x[:, rank * vl:(rank + 1) * vl].copy()), md,
                                             noise_shard=torch.from_numpy(noise[:, rank * vl:(rank + 1) * vl].copy()),
                                             k_cand=32, exchange=ex)
        assert ex.args == (rank * vl, V)
        assert tok2.tolist() == tok.tolist()
        q.put((rank, tok.numpy().tolist()))
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_plumbing_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    B, V = 12, 4096
    x, _, tp, T, noise = o.make_sharded_inputs(B=B, V=V, seed=4, dtype="f32")
    tk = np.random.default_rng(0).integers(1, 33, B).astype(np.int32)
    expected = o.sample(x, tk, tp, T, noise=noise).tolist()
    assert got[0] == got[1] == expected   # every rank ends with the unsharded answer


def test_batch_shards_reproduce_the_unsharded_tokens():
    # rows r0.. of a batch sampled alone with dim0_offset = r0 equal the same rows of the whole batch
    x, tk, tp, T, _ = o.make_sampling_inputs(B=8, V=2048, seed=3, dtype="f32")
    key = (11, 22)
    whole = o.sample(x, tk, tp, T, rng_key=key)
    for r0 in (0, 4):
        part = o.sample(x[r0:r0 + 4], tk[r0:r0 + 4], tp[r0:r0 + 4], T[r0:r0 + 4], rng_key=key, dim0_offset=r0)
        assert np.array_equal(part, whole[r0:r0 + 4])
