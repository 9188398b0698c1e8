"""Sampling namespace (mirror of tallax/sampling.py:8-18).

The reference re-exports two names that do not exist in its own source; the two
that do exist are kept, and the one-call sampler entry points are added.
"""
from tallax_b200._src.sampling import top_p_mask as top_p_mask
from tallax_b200._src.sampling import top_p_and_sample as top_p_and_sample
from tallax_b200._src.sampling import sample as sample
from tallax_b200._src.sampling import sample_vocab_sharded as sample_vocab_sharded
from tallax_b200._src.sampling import VocabShardedWorkspace as VocabShardedWorkspace
from tallax_b200._src.sampling import make_vocab_exchange as make_vocab_exchange
from tallax_b200._src.sampling import SamplingMetadata as SamplingMetadata

__all__ = ["top_p_mask", "top_p_and_sample", "sample", "sample_vocab_sharded", "VocabShardedWorkspace",
           "make_vocab_exchange", "SamplingMetadata"]
