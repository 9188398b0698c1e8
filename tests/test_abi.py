"""CPU checks of the drop-in boundary: the library loads and exports every declared symbol."""
import os
import re

from tallax_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tallax_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tlx_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    build.build()
    lib = _lib.load()
    assert lib.tlx_abi_version() == 1


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    # bad axis is rejected before any CUDA call
    rc = lib.tlx_cumsum(None, None, None, 4, 4, _lib.TLX_F32, 2, 0)
    assert rc == _lib.TLX_ERR_INVALID
    assert b"axis" in lib.tlx_last_error()
    rc = lib.tlx_top_k(None, None, _lib.TLX_F32, 4, 100, 100, 4096, None, 0, 0.0, 0, None, None, None, None, None,
                       None, 0)
    assert rc == _lib.TLX_ERR_UNSUPPORTED
    assert lib.tlx_sort_workspace_bytes(128, 65536) == 128 * 65536 * 8
    assert lib.tlx_sort_workspace_bytes(16, 2048) == 0
    assert lib.tlx_sample_workspace_bytes(256, 128256) > 256 * 4
    assert lib.tlx_sample_workspace_bytes(0, 128256) == 0


def test_python_mirror_error_behaviour():
    import pytest
    import torch

    from tallax_b200 import tax, tumpy
    from tallax_b200._src.bitonic_top_k import bitonic_top_k
    from tallax_b200._src.sampling import top_p_mask

    a = torch.zeros(2, 2, 16)
    with pytest.raises(ValueError):
        tumpy.sort(a, axis=0)
    with pytest.raises(ValueError):
        tax.sort([torch.zeros(2, 4), torch.zeros(2, 5)], num_keys=1)
    with pytest.raises(ValueError):
        tax.sort(torch.zeros(4), num_keys=1)
    with pytest.raises(ValueError):
        bitonic_top_k(torch.zeros(8, 256), k=256)
    with pytest.raises(NotImplementedError):
        bitonic_top_k(torch.zeros(8, 256), k=128, descending=False)
    with pytest.raises(ValueError):
        tax.top_k(torch.zeros(7, 256), 4)  # num_tokens not divisible by block_token
    with pytest.raises(NotImplementedError):
        tax.top_dynamic_k(torch.zeros(8, 8192), k=4, max_k=4096)
    with pytest.raises(NotImplementedError):
        top_p_mask(topk_logits=torch.zeros(4, 4), p=torch.zeros(4), replace_val=0.0, axis=1)
    with pytest.raises(ValueError):
        tax.cumsum(torch.zeros(4, 4), axis=0)  # CPU tensor: there is no CPU path


def test_xla_ffi_adapter_compiles_without_xla_and_binds_declared_symbols(tmp_path):
    import shutil
    import subprocess
    src = os.path.join(ROOT, "tallax_b200", "ffi", "xla_ffi_adapter.cc")
    text = open(src).read()
    used = set(re.findall(r"\b(tlx_[a-z0-9_]+)\s*\(", re.sub(r"//.*", "", text)))
    assert {"tlx_sample_dev", "tlx_top_p_and_sample_dev", "tlx_gumbel_argmax_dev", "tlx_sparse_random_uniform_dev",
            "tlx_shard_candidates_dev"} <= used
    assert used <= set(_declared()), used - set(_declared())
    gxx = shutil.which("g++")
    if gxx:   # no XLA headers here: the guard leaves an empty object
        obj = str(tmp_path / "ffi.o")
        subprocess.run([gxx, "-std=c++17", "-fPIC", "-I", os.path.join(ROOT, "include"), "-c", src, "-o", obj], check=True)


def test_device_operand_entry_points_reject_missing_key_without_gpu():
    lib = _lib.load()
    rc = lib.tlx_sample_dev(None, None, _lib.TLX_BF16, 4, 128256, 128256, None, None, None, None, 0, None, None, None,
                            None, None, 0)
    assert rc == _lib.TLX_ERR_INVALID and b"key" in lib.tlx_last_error()
    rc = lib.tlx_gumbel_argmax_dev(None, None, None, None, 4, 4, None, 16, 1, None)
    assert rc == _lib.TLX_ERR_INVALID


def test_exchange_layout_and_argument_errors_need_no_gpu():
    import ctypes
    lib = _lib.load()
    # header (256 B) + two sets of (arrival words, world * 3 * rows * k floats), each padded to 256 B
    rows, k, world = 1024, 50, 8
    flags = (rows * 4 + 255) // 256 * 256
    cand = (world * 3 * rows * k * 4 + 255) // 256 * 256
    assert lib.tlx_exchange_bytes(rows, k, world) == 256 + 2 * (flags + cand)
    assert lib.tlx_exchange_bytes(rows, k, 17) == 0 and lib.tlx_exchange_bytes(0, k, 2) == 0
    bufs = (ctypes.c_void_p * 2)(None, None)
    # rank outside the world, and a missing buffer: rejected before any CUDA call
    rc = lib.tlx_exchange_shard_candidates(None, None, _lib.TLX_BF16, 4, 64, 64, 0, 8, None, 0, None, 0, 0, 128, 0, None,
                                           2, 2, bufs)
    assert rc == _lib.TLX_ERR_INVALID and b"rank" in lib.tlx_last_error()
    rc = lib.tlx_exchange_shard_candidates(None, None, _lib.TLX_BF16, 4, 64, 64, 0, 8, None, 0, None, 0, 0, 128, 0, None,
                                           0, 2, bufs)
    assert rc == _lib.TLX_ERR_INVALID and b"buffer of rank 0" in lib.tlx_last_error()
    rc = lib.tlx_exchange_merge_and_sample(None, None, 4, 8, 2, None, None, None, None, None)
    assert rc == _lib.TLX_ERR_INVALID
    rc = lib.tlx_exchange_merge_and_sample(None, None, 4, 1024, 16, None, None, None, None, None)
    assert rc == _lib.TLX_ERR_UNSUPPORTED
