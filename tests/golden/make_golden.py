"""Generates tests/golden/*.npz by running the REFERENCE's own value-level functions.

    python tests/golden/make_golden.py /path/to/reference/checkout

The reference (oliverdutton/tallax) is imported from the given checkout with `jax.numpy`
mapped onto NumPy (jax_numpy_shim.py); nothing of it is copied.  Each fixture stores the
seeded inputs and the reference function's outputs; tests/test_golden.py checks the oracle and
(on a GPU) the CUDA library against them.  Re-run only when the reference changes.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)


def main(ref_root: str):
    import jax_numpy_shim

    jax_numpy_shim.install()
    sys.path.insert(0, ref_root)
    from tallax._src import utils as rutils
    from tallax._src.cumsum import cumsum_arrays
    from tallax._src.gather import take_along_axis_arrays
    from tallax._src.bitonic_top_k import max_arrays
    from tallax._src.sparse_random import sparse_random_uniform, sparse_random_categorical
    from tallax._src.sampling import top_p_mask, top_p_and_sample_arrays

    rng = np.random.Generator(np.random.Philox(20240))
    out = {}
    J = jax_numpy_shim.as_jax   # arrays handed to the reference get jax's value semantics

    # --- key transform: utils.py:139-200 --------------------------------------------------------
    x = rng.standard_normal(512).astype(np.float32) * 4
    x[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 3.0]
    out["key_in"] = x
    out["key_sortable_int"] = rutils.float_to_sortable_int(J(x))
    out["key_roundtrip"] = rutils.sortable_int_to_float(J(out["key_sortable_int"]))

    # --- cumsum_arrays: cumsum.py:32-63 -----------------------------------------------------------
    for i, (shape, axis, rev) in enumerate([((8, 128), 1, False), ((16, 256), 0, True), ((13, 167), 1, True),
                                            ((128, 8), 0, False), ((13, 167), 0, False)]):
        a = rng.standard_normal(shape).astype(np.float32)
        ai = rng.integers(0, 100, shape).astype(np.int32)
        out[f"cumsum{i}_f32_in"], out[f"cumsum{i}_i32_in"] = a, ai
        out[f"cumsum{i}_meta"] = np.array([axis, int(rev)])
        out[f"cumsum{i}_f32_out"] = cumsum_arrays(J(a), axis=axis, reverse=rev)
        out[f"cumsum{i}_i32_out"] = cumsum_arrays(J(ai), axis=axis, reverse=rev)

    # --- take_along_axis_arrays: gather.py:11-45 (with out-of-range indices) -------------------------
    for i, (vshape, k, axis) in enumerate([((8, 300), 200, 1), ((13, 256), 64, 1), ((300, 16), 128, 0)]):
        v = rng.standard_normal(vshape).astype(np.float32)
        n = vshape[axis]
        ishape = (vshape[0], k) if axis == 1 else (k, vshape[1])
        idx = rng.integers(-5, n + 5, ishape).astype(np.int32)
        out[f"gather{i}_val"], out[f"gather{i}_idx"], out[f"gather{i}_axis"] = v, idx, np.array(axis)
        out[f"gather{i}_out"] = take_along_axis_arrays(J(v), J(idx), axis)

    # --- max_arrays: bitonic_top_k.py:43-97 -------------------------------------------------------------
    for i, (shape, axis) in enumerate([((16, 256), 1), ((173, 195), 1), ((128, 8), 0), ((256, 16), 0)]):
        v = rng.standard_normal(shape).astype(np.float32)   # continuous values: no ties, so the winner is unique
        iota = np.broadcast_to(np.arange(shape[axis], dtype=np.int32).reshape((-1, 1) if axis == 0 else (1, -1)),
                               shape).copy()
        r = max_arrays([J(v), J(iota)], num_keys=1, axis=axis)
        out[f"max{i}_val"], out[f"max{i}_axis"] = v, np.array(axis)
        out[f"max{i}_out_val"], out[f"max{i}_out_idx"] = np.asarray(r[0]), np.asarray(r[1])

    # --- sparse_random_uniform: sparse_random.py:43-64 -----------------------------------------------------
    for i, (seed, lo, hi) in enumerate([((42, 7), 0.0, 1.0), ((123, 456), -1.0, 1.0), ((9, 9), 5.0, 10.0)]):
        key = np.array([seed], np.uint32)   # (1, 2) key as the kernel receives it
        i0 = rng.integers(0, 16, (8, 128)).astype(np.int32)
        i1 = rng.integers(0, 256, (8, 128)).astype(np.int32)
        out[f"uniform{i}_key"], out[f"uniform{i}_i0"], out[f"uniform{i}_i1"] = key, i0, i1
        out[f"uniform{i}_range"] = np.array([lo, hi], np.float32)
        out[f"uniform{i}_out"] = sparse_random_uniform(J(key), [J(i0), J(i1)], dim1_size=256, minval=lo, maxval=hi)

    # --- top_p_mask: sampling.py:25-62, on the (k, B) layout -------------------------------------------------
    x = -np.sort(-rng.standard_normal((128, 32)).astype(np.float32) * 3, axis=0)
    p = rng.uniform(0.05, 0.999, 32).astype(np.float32)
    out["topp_in"], out["topp_p"] = x, p
    out["topp_out"] = top_p_mask(topk_logits=J(x), p=J(p), replace_val=-1e12, axis=0)

    # --- top_p_and_sample_arrays: sampling.py:65-115 ------------------------------------------------------------
    B, k, V = 32, 128, 50000
    logits = rng.standard_normal((B, V)).astype(np.float32) * 3
    order = np.argsort(-logits, axis=1, kind="stable")[:, :k]
    vals = np.take_along_axis(logits, order, 1)
    kk = rng.integers(1, k + 1, B)
    vals[np.arange(k)[None, :] >= kk[:, None]] = np.float32(-1e12)
    top_p = rng.uniform(0.5, 0.99, B).astype(np.float32)
    temp = rng.uniform(0.5, 1.5, B).astype(np.float32)
    temp[3] = 0.0
    key = np.array([[77, 1234]], np.uint32)
    tok = top_p_and_sample_arrays(topk_logits=J(vals), topk_idx=J(order.astype(np.int32)), rng_key=J(key), top_p=J(top_p),
                                  temperature=J(temp), vocab_size=V, replace_val=-1e12, dim0_offset=5)
    out["sample_vals"], out["sample_idx"] = vals, order.astype(np.int32)
    out["sample_top_p"], out["sample_temp"], out["sample_key"] = top_p, temp, key
    out["sample_meta"] = np.array([V, 5])
    out["sample_tokens"] = np.asarray(tok).astype(np.int32)

    # --- sparse_random_categorical: sparse_random.py:68-94, axis 1 -------------------------------------------------
    lg = rng.standard_normal((16, 128)).astype(np.float32)
    cols = np.stack([rng.choice(256, 128, replace=False) for _ in range(16)]).astype(np.int32)
    rws = np.broadcast_to(np.arange(16, dtype=np.int32)[:, None], (16, 128)).copy()
    r = sparse_random_categorical(J(np.array([[5, 6]], np.uint32)), J(lg), [J(rws), J(cols)], dim1_size=256, axis=1)
    out["cat_logits"], out["cat_rows"], out["cat_cols"] = lg, rws, cols
    out["cat_out0"], out["cat_out1"] = np.asarray(r[0]).astype(np.int32), np.asarray(r[1]).astype(np.int32)

    # --- compare_and_swap: sort.py:39-102 ---------------------------------------------------------------
    # (a) pairs of columns, key + payload, every direction form the function takes
    from tallax._src.sort import compare_and_swap
    kl = rng.integers(-4, 5, (4, 256)).astype(np.float32)          # small integers: many ties
    kr = rng.integers(-4, 5, (4, 256)).astype(np.float32)
    kl[0, :4] = [0.0, -0.0, 1.0, 2.0]
    kr[0, :4] = [-0.0, 0.0, 1.0, 2.0]
    pl_ = np.arange(4 * 256, dtype=np.int32).reshape(4, 256)        # payload = unique id, lefts below rights
    pr_ = pl_ + 4 * 256
    dyn = rng.integers(0, 2, (4, 256)).astype(np.int32)
    out["cas_kl"], out["cas_kr"], out["cas_pl"], out["cas_pr"], out["cas_dyn"] = kl, kr, pl_, pr_, dyn
    for name, nk, desc in (("asc1", 1, False), ("desc1", 1, True), ("asc2", 2, False), ("desc2", 2, True),
                           ("dyn1", 1, J(dyn)), ("dyn2", 2, J(dyn))):
        (ol_k, or_k), (ol_p, or_p) = compare_and_swap((J(kl), J(pl_)), (J(kr), J(pr_)), num_keys=nk, is_descending=desc)
        out[f"cas_{name}_lk"], out[f"cas_{name}_rk"] = np.asarray(ol_k), np.asarray(or_k)
        out[f"cas_{name}_lp"], out[f"cas_{name}_rp"] = np.asarray(ol_p), np.asarray(or_p)
    # (b) a whole bitonic network over rows of 64 made of nothing but that comparator, keys (value, column)
    n = 64
    v = rng.integers(-6, 7, (8, n)).astype(np.float32)
    v[1] = 3.0
    v[2, ::2] = -0.0
    v[2, 1::2] = 0.0
    col = np.broadcast_to(np.arange(n, dtype=np.int32), (8, n)).copy()
    for name, desc in (("asc", False), ("desc", True)):
        a, b = v.copy(), col.copy()
        size = 2
        while size <= n:
            stride = size // 2
            while stride >= 1:
                i = np.arange(n)
                lo = i[(i & stride) == 0]
                hi = lo | stride
                up = ((lo & size) == 0)[None, :]                  # sub-sequence direction of the bitonic network
                d = np.broadcast_to(up != (not desc), (8, len(lo))).astype(np.int32)   # 1 = descending pair
                (la, ra), (lb, rb) = compare_and_swap((J(a[:, lo]), J(b[:, lo])), (J(a[:, hi]), J(b[:, hi])), num_keys=2,
                                                      is_descending=J(d))
                a[:, lo], a[:, hi], b[:, lo], b[:, hi] = np.asarray(la), np.asarray(ra), np.asarray(lb), np.asarray(rb)
                stride //= 2
            size *= 2
        out[f"net_{name}_val"], out[f"net_{name}_col"] = a, b
    out["net_in"] = v

    # --- binned_top_k: top_k.py:13-106 (a ragged last slice; ties inside a bin) ------------------------------
    from tallax._src.top_k import binned_top_k
    kb, nb = 4, 128
    xb = rng.integers(-20, 21, (4, 1000)).astype(np.float32)        # integers: ties inside most bins
    xb[1] = rng.standard_normal(1000).astype(np.float32)
    vals0 = [J(np.full((4, nb), np.finfo(np.float32).min, np.float32)) for _ in range(kb)]
    idxs0 = [J(np.zeros((4, nb), np.int32)) for _ in range(kb)]
    bv, bi = binned_top_k(J(xb), kb, vals0, idxs0, num_bins=nb)
    out["binned_in"] = xb
    out["binned_vals"] = np.stack([np.asarray(t) for t in bv])
    out["binned_idxs"] = np.stack([np.asarray(t) for t in bi])

    # --- pack_bf16_u16_to_i32 / unpack: utils.py:205-227 ------------------------------------------------------
    import ml_dtypes
    xp = (rng.integers(-8, 9, (4, 512)).astype(np.float32) * 0.5).astype(ml_dtypes.bfloat16)
    xp[0, :4] = np.array([0.0, -0.0, 1.0, -1.0], np.float32).astype(ml_dtypes.bfloat16)
    xp[3] = (rng.standard_normal(512).astype(np.float32) * 3).astype(ml_dtypes.bfloat16)
    ip = np.broadcast_to(np.arange(512, dtype=np.int32), (4, 512)).copy()
    packed = rutils.pack_bf16_u16_to_i32(J(xp), J(ip))
    uv, ui = rutils.unpack_bf16_u16_from_i32(J(np.asarray(packed)))
    out["pack_in"] = xp.astype(np.float32)    # bf16 values, stored as f32 (npz has no bf16)
    out["pack_packed"] = np.asarray(packed).astype(np.int32)
    out["pack_unpacked_val"] = np.asarray(uv).astype(np.float32)
    out["pack_unpacked_idx"] = np.asarray(ui).astype(np.int32)

    path = os.path.join(HERE, "reference_value_level.npz")
    np.savez_compressed(path, **{k: np.asarray(v) for k, v in out.items()})
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of oliverdutton/tallax>")
    main(sys.argv[1])
