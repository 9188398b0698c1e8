"""tallax_b200: B200-native (sm_100a) row-wise top-k / sort / gather / cumsum / fused sampling.

The public modules keep the names and signatures of the reference project's
`tax`, `tumpy` and `sampling` namespaces; arrays are torch CUDA tensors.
"""
from tallax_b200 import tax
from tallax_b200 import tumpy
from tallax_b200 import sampling

__all__ = ["tax", "tumpy", "sampling"]
