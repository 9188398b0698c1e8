"""lax-like namespace (mirror of tallax/tax.py:13-23): sort, top_k, top_dynamic_k, cumsum."""
from tallax_b200._src.sort import sort as sort
from tallax_b200._src.top_k import top_k as top_k
from tallax_b200._src.top_k import top_dynamic_k as top_dynamic_k
from tallax_b200._src.cumsum import cumsum as cumsum

__all__ = ["sort", "top_k", "top_dynamic_k", "cumsum"]
