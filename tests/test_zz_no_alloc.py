"""The allocation-free sort entry point against the regular one.

tlx_sort_static is for callers that cannot provide scratch memory (no cudaMalloc allowed in
their position: under a foreign memory pool, or on a fixed budget);
it keeps the scratch in a fixed area inside the library.  It must give exactly what tlx_sort
gives, call after call, since every call reuses the same area.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sort_both(lib, torch, keys, descending):
    from tallax_b200 import _lib

    rows, n = keys.shape
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        out_keys = torch.empty_like(keys)
        out_perm = torch.empty((rows, n), dtype=torch.int32, device=keys.device)
        if static:
            rc = lib.tlx_sort_static(stream, keys.data_ptr(), _lib.TLX_F32, rows, n, int(descending), None,
                                     out_keys.data_ptr(), out_perm.data_ptr())
        else:
            ws = torch.empty(max(lib.tlx_sort_workspace_bytes(rows, n), 16), dtype=torch.uint8, device=keys.device)
            rc = lib.tlx_sort(stream, keys.data_ptr(), _lib.TLX_F32, rows, n, int(descending), None,
                              out_keys.data_ptr(), out_perm.data_ptr(), ws.data_ptr(), ws.numel())
        assert rc == 0, lib.tlx_last_error()
        torch.cuda.synchronize()
        outs.append((out_keys.cpu().numpy(), out_perm.cpu().numpy()))
    return outs


def test_static_sort_matches_regular_sort_twice_in_a_row(cuda):
    import torch

    from tallax_b200 import _lib

    lib = _lib.load()
    assert lib.tlx_sort_static_max_bytes() == 16 << 20
    rng = np.random.default_rng(7)
    # two different problems back to back: the second call finds the first one's leftovers in the area
    for rows, n, descending in ((6, 65536, False), (3, 100000, True), (16, 2048, False)):
        keys = rng.standard_normal((rows, n)).astype(np.float32)
        keys[:, ::97] = keys[:, 5:6]   # ties: the permutation must still be the stable one
        (k0, p0), (k1, p1) = _sort_both(lib, torch, torch.from_numpy(keys).to(cuda), descending)
        assert np.array_equal(k0, k1) and np.array_equal(p0, p1)   # integer / bit-exact work: no tolerance
        order = np.argsort(-keys if descending else keys, axis=1, kind="stable")
        assert np.array_equal(p1, order)


def test_static_sort_rejects_what_does_not_fit(cuda):
    import torch

    from tallax_b200 import _lib

    lib = _lib.load()
    keys = torch.zeros((64, 65536), device=cuda)   # 64 * 65536 * 8 bytes = 32 MiB of composites > 16 MiB
    out = torch.empty((64, 65536), dtype=torch.int32, device=cuda)
    rc = lib.tlx_sort_static(torch.cuda.current_stream().cuda_stream, keys.data_ptr(), _lib.TLX_F32, 64, 65536, 0,
                             None, None, out.data_ptr())
    assert rc == _lib.TLX_ERR_INVALID
    assert b"built-in area" in lib.tlx_last_error()
