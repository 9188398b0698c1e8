"""Fused sampler (mirror of tallax/_src/sampling.py:25-343)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from tallax_b200._src import ops

_SAMPLING_EPS = 1e-5
_REPLACE_VAL = -1e12


@dataclass
class SamplingMetadata:
    """The three per-request vectors `sample` reads from its metadata argument
    (sampling.py:335-341).  Any object with these attributes works."""
    top_k: Any
    top_p: Any
    temperature: Any


def top_p_mask(*, topk_logits, p, replace_val, axis):
    """Top-p filter on candidates sorted descending along axis 0, shape (k, batch)
    (sampling.py:25-62): softmax on the unscaled logits, threshold index = number of
    cumulative masses below p, ties at the threshold kept."""
    if axis != 0:
        raise NotImplementedError("topp_mask only supports axis=0")
    return ops.top_p_mask(topk_logits, p, replace_val)


def top_p_and_sample(topk_logits, topk_idx, rng_key, top_p, temperature, *, vocab_size, replace_val,
                     interpret: bool = False, noise=None, dim0_offset: int = 0):
    """Top-p, temperature and Gumbel arg-max on [batch, k] candidates sorted descending whose
    masked tail already holds `replace_val` (sampling.py:214-269).  Returns int32 [batch].

    `rng_key` is the two-word threefry key; the keyword-only `noise` (dense float32
    [batch_total, vocab] uniforms) replaces it when given.  `dim0_offset` is the first
    global row of a batch shard (sampling.py:248-258).
    """
    return ops.top_p_and_sample(topk_logits, topk_idx, top_p, temperature, vocab_size=vocab_size,
                                replace_val=replace_val, rng_key=rng_key, noise=noise, dim0_offset=dim0_offset)


def sample(rng_key, logits, tpu_sampling_metadata, *, noise=None, dim0_offset: int = 0, workspace=None):
    """The decode sampler vLLM calls (sampling.py:331-343): logits [batch, vocab] -> int32 [batch].

    One fused call replaces the reference's top-k kernel + sampling kernel.  top_k <= 0 or
    >= vocab disables the top-k filter (an extension; the reference supports 1..128 only).
    """
    md = tpu_sampling_metadata
    return ops.sample(logits, md.top_k, md.top_p, md.temperature, rng_key=rng_key, noise=noise,
                      dim0_offset=dim0_offset, workspace=workspace)


class VocabShardedWorkspace:
    """Preallocated buffers of `sample_vocab_sharded` (this rank's candidate block, the gathered blocks of all
    ranks, the tokens), so that a decode loop allocates nothing per step."""

    def __init__(self, rows: int, k_cand: int, world: int, device):
        self.rows, self.k_cand, self.world = rows, k_cand, world
        self.gathered = torch.empty((world, 3, rows, k_cand), dtype=torch.float32, device=device)
        self.block = torch.empty((3, rows, k_cand), dtype=torch.float32, device=device)
        self.tokens = torch.empty(rows, dtype=torch.int32, device=device)


def make_vocab_exchange(rows: int, k_cand: int, group=None, device=None):
    """This rank's exchange buffer for `sample_vocab_sharded(..., exchange=...)`, with the other ranks' buffers
    mapped: every rank of `group` calls it with the same `rows` and `k_cand` (a collective: the handles are
    all-gathered and a barrier ends it).  Keep it for the life of the decode loop; `.close()` frees it."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    ex = ops.Exchange.create(rows, k_cand, world, device)
    handles = [None] * world
    if world > 1:
        dist.all_gather_object(handles, ex.handle, group=group)
    else:
        handles = [ex.handle]
    ex.attach(rank, handles)
    if world > 1:
        dist.barrier(group=group)
    return ex


def sample_vocab_sharded(rng_key, logits_shard, tpu_sampling_metadata, *, group=None, noise_shard=None,
                         k_cand: int | None = None, dim0_offset: int = 0, workspace=None, exchange=None):
    """Sampler for logits sharded along the vocabulary across the ranks of `group`
    (the shard-mapped body of sampling.py:300-321): local top-k' on this rank's
    contiguous slice, one all-gather of the (value, global token, noise) candidates,
    then merge and sample.  Every rank returns the same tokens.

    Needs 1 <= top_k <= k_cand for every row (the reference fixes k' = 128).
    One library call per stage; with `workspace` (a VocabShardedWorkspace) nothing is allocated.

    With `exchange` (from `make_vocab_exchange`) there is no collective call: the candidate kernel stores
    every row's block into all ranks' exchange buffers over NVLink and the merge kernel waits per row for
    the blocks to arrive.  `workspace.tokens`, when given, receives the result.
    """
    import torch.distributed as dist

    md = tpu_sampling_metadata
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    rows, v_local = logits_shard.shape
    if exchange is not None:
        if exchange.world != world or exchange.rank != rank:
            raise ValueError("exchange was made for another group")
        ops.exchange_shard_candidates(logits_shard, rank * v_local, exchange, noise_shard=noise_shard, rng_key=rng_key,
                                      vocab_total=v_local * world, dim0_offset=dim0_offset)
        return ops.exchange_merge_and_sample(exchange, md.top_k, md.top_p, md.temperature,
                                             out=workspace.tokens if workspace is not None else None)
    if k_cand is None:
        k_cand = 128
    k_cand = min(k_cand, v_local)
    w = workspace
    if w is None:
        w = VocabShardedWorkspace(rows, k_cand, world, logits_shard.device)
    elif (w.rows, w.k_cand, w.world) != (rows, k_cand, world):
        raise ValueError("workspace was made for another shape")
    # a single rank writes its block straight into the gathered buffer
    block = w.gathered[0] if world == 1 else w.block
    ops.shard_candidates(logits_shard, rank * v_local, k_cand, noise_shard=noise_shard, rng_key=rng_key,
                         vocab_total=v_local * world, dim0_offset=dim0_offset, out=block)
    if world > 1:
        # concatenated-along-dim-0 form: the one every backend accepts
        dist.all_gather_into_tensor(w.gathered.view((world * 3,) + tuple(block.shape[1:])), block, group=group)
    return ops.merge_and_sample(w.gathered, md.top_k, md.top_p, md.temperature, out=w.tokens)
