"""ctypes binding of libtallax_b200.so (the C ABI declared in include/tallax_b200.h).

There is no fallback: if the library is missing every operator raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libtallax_b200.so")

TLX_F32, TLX_BF16, TLX_I32, TLX_F16, TLX_U32 = 0, 1, 2, 3, 4
TLX_OK, TLX_ERR_INVALID, TLX_ERR_UNSUPPORTED, TLX_ERR_WORKSPACE, TLX_ERR_CUDA = 0, -1, -2, -3, -4
TOPK_MAX_K = 2048

_vp, _i64, _i32, _u32, _f32, _f64, _sz = (C.c_void_p, C.c_int64, C.c_int, C.c_uint32, C.c_float, C.c_double,
                                          C.c_size_t)

# name -> (restype, argtypes); must list every symbol include/tallax_b200.h declares
SIGNATURES = {
    "tlx_abi_version": (_i32, []),
    "tlx_last_error": (C.c_char_p, []),
    "tlx_kernel_launches": (C.c_ulonglong, []),
    "tlx_init": (_i32, [_i32, _u32]),
    "tlx_debug_check_status": (_i32, [_vp]),
    "tlx_take_along_axis": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32]),
    "tlx_cumsum": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32]),
    "tlx_argmax": (_i32, [_vp, _vp, _i32, _i64, _i64, _i32, _vp]),
    "tlx_sort_workspace_bytes": (_sz, [_i64, _i64]),
    "tlx_sort": (_i32, [_vp, _vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _sz]),
    "tlx_sort_static_max_bytes": (_sz, []),
    "tlx_sort_static": (_i32, [_vp, _vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp]),
    "tlx_top_k_workspace_bytes": (_sz, [_i64, _i64, _i32]),
    "tlx_top_k": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i32, _vp, _i32, _f64, _i32, _vp, _vp, _vp, _vp, _vp,
                         _vp, _sz]),
    "tlx_canonicalize_keys": (_i32, [_vp, _vp, _i32, _i64]),
    "tlx_sparse_random_uniform": (_i32, [_vp, _u32, _u32, _vp, _vp, _i64, _i64, _f32, _f32, _vp]),
    "tlx_sparse_random_uniform_dev": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _f32, _vp]),
    "tlx_gumbel_argmax_dev": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i32, _vp]),
    "tlx_top_p_and_sample_dev": (_i32, [_vp, _vp, _i32, _vp, _i64, _i32, _vp, _vp, _vp, _i64, _vp, _i64, _f64, _vp,
                                        _vp]),
    "tlx_sample_dev": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp,
                              _sz]),
    "tlx_shard_candidates_dev": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i64, _vp,
                                        _vp, _vp, _vp, _vp, _sz]),
    "tlx_top_p_mask": (_i32, [_vp, _vp, _vp, _i32, _i64, _f64, _vp]),
    "tlx_gumbel_argmax": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _u32, _u32, _i64, _i32, _vp]),
    "tlx_top_p_and_sample": (_i32, [_vp, _vp, _i32, _vp, _i64, _i32, _vp, _vp, _vp, _i64, _u32, _u32, _i64, _f64,
                                    _i64, _vp]),
    "tlx_sample_workspace_bytes": (_sz, [_i64, _i64]),
    "tlx_sample": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _u32, _u32, _i64, _vp, _vp,
                          _vp, _sz]),
    "tlx_shard_candidates_workspace_bytes": (_sz, [_i64, _i64, _i32]),
    "tlx_shard_candidates": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _u32, _u32, _i64, _i64,
                                    _vp, _vp, _vp, _vp, _sz]),
    "tlx_merge_and_sample": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _i64, _vp, _vp, _vp, _vp]),
    "tlx_exchange_bytes": (_sz, [_i64, _i32, _i32]),
    "tlx_exchange_create": (_i32, [_i64, _i32, _i32, _vp, _vp]),
    "tlx_exchange_open": (_i32, [_vp, _vp]),
    "tlx_exchange_close": (_i32, [_vp]),
    "tlx_exchange_destroy": (_i32, [_vp]),
    "tlx_exchange_status": (_i32, [_vp, _vp, _vp, _vp]),
    "tlx_exchange_shard_candidates": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _u32, _u32,
                                             _i64, _i64, _vp, _i32, _i32, _vp]),
    "tlx_exchange_merge_and_sample": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
}

_lib = None


class TallaxLibraryError(RuntimeError):
    pass


def load():
    """Loads the shared library (once) and attaches the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_PATH
    if os.environ.get("TLX_LIBRARY") == "checked":   # the index-checking build (python -m tallax_b200.build --checked)
        path = os.path.join(os.path.dirname(LIB_PATH), "libtallax_b200_checked.so")
    if not os.path.exists(path):
        raise TallaxLibraryError(
            f"{path} is missing: build it with `python -m tallax_b200.build`; there is no CPU or PyTorch fallback")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.tlx_abi_version() != 1:
        raise TallaxLibraryError("libtallax_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def check(rc: int):
    """Maps a status code to the exception class the reference raises for that kind of error."""
    if rc == TLX_OK:
        return
    msg = load().tlx_last_error().decode()
    if rc == TLX_ERR_INVALID:
        raise ValueError(msg)
    if rc == TLX_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"tallax_b200 error {rc}: {msg}")
