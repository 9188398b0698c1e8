"""GPU: the streaming sampler under the index-checking build (python -m tallax_b200.build --checked).

The checked library verifies the shared-memory and workspace indices the kernels rely on and records the first
one out of range; it stands in for a memory checker.  A child process loads it (TLX_LIBRARY=checked), runs the
sampler over inputs that reach its different row classes, and reports the record.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes, json, sys
import numpy as np, torch
sys.path.insert(0, %r)
from oracle import tallax_oracle as o
from tallax_b200 import _lib
from tallax_b200._src import ops
from tests.conftest import to_dev, to_np
lib = _lib.load()
cuda = torch.device("cuda", 0)
bad = 0
for B, V, seed in ((48, 128256, 2), (300, 32768, 5), (16, 151936, 6)):
    x, tk, tp, T, noise = o.make_sampling_inputs(B=B, V=V, seed=seed, dtype="bf16")
    tk[::7] = 0            # rows without top-k: histogram and final items
    tk[1::7] = 1024
    T[2] = 0.0             # a greedy row
    tp[3] = 1.0
    exp, flags = o.sample(x, tk, tp, T, noise=noise, return_flags=True)
    tok = ops.sample(to_dev(x, cuda), to_dev(tk, cuda), to_dev(tp, cuda), to_dev(T, cuda), noise=to_dev(noise, cuda))
    bad += int(((to_np(tok) != exp) & ~flags).sum())
    tok = ops.sample(to_dev(x, cuda), to_dev(tk, cuda), to_dev(tp, cuda), to_dev(T, cuda), rng_key=(1, 2))
w = (ctypes.c_int32 * 4)()
rc = lib.tlx_debug_check_status(w)
print(json.dumps({"rc": rc, "word": list(w), "mismatches": bad}))
"""


def test_streaming_sampler_passes_its_index_checks(cuda):
    lib = os.path.join(ROOT, "tallax_b200", "lib", "libtallax_b200_checked.so")
    if not os.path.exists(lib):
        from tallax_b200 import build
        build.build(checked=True)
    env = dict(os.environ, TLX_LIBRARY="checked")
    res = subprocess.run([sys.executable, "-c", CHILD % ROOT], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rec = json.loads(res.stdout.strip().splitlines()[-1])
    assert rec["rc"] == 0 and rec["word"][0] == 0, rec      # no index out of range
    assert rec["mismatches"] == 0


def test_normal_build_says_it_is_not_checked(cuda):
    from tallax_b200 import _lib
    lib = _lib.load()
    assert lib.tlx_debug_check_status(None) == _lib.TLX_ERR_UNSUPPORTED
