"""Thin tensor-level wrappers over the C ABI.

PyTorch is used for device memory and streams only: every function allocates its
outputs (and workspace) as torch CUDA tensors and passes raw pointers plus the current
stream to libtallax_b200.so.
"""
from __future__ import annotations

import torch

from tallax_b200 import _lib
from tallax_b200._lib import check

_DT = {
    torch.float32: _lib.TLX_F32,
    torch.bfloat16: _lib.TLX_BF16,
    torch.int32: _lib.TLX_I32,
    torch.float16: _lib.TLX_F16,
}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise NotImplementedError(f"dtype {t.dtype} is not supported") from None


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _dev(t: torch.Tensor) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError("expected a torch.Tensor on a CUDA device")
    if not t.is_cuda:
        raise ValueError("tallax_b200 operators need CUDA tensors; there is no CPU path")
    return t.contiguous()


def _ws(nbytes: int, device) -> torch.Tensor | None:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _i32vec(v, rows: int, device) -> torch.Tensor:
    if isinstance(v, torch.Tensor):
        v = v.to(device=device, dtype=torch.int32)
    else:
        v = torch.as_tensor(v, dtype=torch.int32, device=device)
    return v.broadcast_to((rows,)).contiguous()


def _f32vec(v, rows: int, device) -> torch.Tensor:
    if isinstance(v, torch.Tensor):
        v = v.to(device=device, dtype=torch.float32)
    else:
        v = torch.as_tensor(v, dtype=torch.float32, device=device)
    return v.broadcast_to((rows,)).contiguous()


def key_pair(rng_key) -> tuple[int, int]:
    """Two uint32 words of a threefry key given as a sequence, numpy array or tensor."""
    if rng_key is None:
        return 0, 0
    if isinstance(rng_key, torch.Tensor):
        rng_key = rng_key.detach().cpu().reshape(-1).tolist()
    else:
        import numpy as np

        rng_key = np.asarray(rng_key).reshape(-1).tolist()
    if len(rng_key) != 2:
        raise ValueError("rng_key must hold two uint32 words")
    return int(rng_key[0]) & 0xFFFFFFFF, int(rng_key[1]) & 0xFFFFFFFF


def key_operand(rng_key):
    """A key that lives on the device (a CUDA tensor of two 32-bit words) is passed to the library as a
    device operand, without a copy to the host; returns that tensor (uint32 view) or None."""
    if isinstance(rng_key, torch.Tensor) and rng_key.is_cuda:
        k = rng_key.detach().reshape(-1)
        if k.numel() != 2 or k.element_size() != 4:
            raise ValueError("a device rng_key must hold two 32-bit words")
        return k.contiguous().view(torch.int32)
    return None


def _host_offset(dim0_offset, dev):
    """A host batch offset for an entry point that takes it as a device operand (None when it is zero)."""
    return None if int(dim0_offset) == 0 else torch.tensor([int(dim0_offset)], dtype=torch.int32, device=dev)


def offset_operand(dim0_offset):
    """A batch offset that lives on the device (a CUDA int32 scalar tensor) stays there; returns it or None."""
    if isinstance(dim0_offset, torch.Tensor) and dim0_offset.is_cuda:
        if dim0_offset.numel() != 1:
            raise ValueError("a device dim0_offset must be a scalar")
        return dim0_offset.detach().reshape(1).to(torch.int32)
    return None


# ---------------------------------------------------------------------------------------
def take_along_axis(values: torch.Tensor, indices: torch.Tensor, axis: int) -> torch.Tensor:
    values, indices = _dev(values), _dev(indices)
    if values.ndim != 2 or indices.ndim != 2:
        raise ValueError("Only 2D inputs supported")
    if indices.dtype != torch.int32:
        indices = indices.to(torch.int32)
    out = torch.empty(indices.shape, dtype=values.dtype, device=values.device)
    check(_lib.load().tlx_take_along_axis(_stream(), _ptr(values), _ptr(indices), _ptr(out), values.shape[0],
                                          values.shape[1], indices.shape[0], indices.shape[1], values.element_size(),
                                          int(axis)))
    return out


def cumsum(arr: torch.Tensor, axis: int, reverse: bool = False) -> torch.Tensor:
    arr = _dev(arr)
    if arr.ndim != 2:
        raise ValueError("Only 2D inputs supported")
    out = torch.empty_like(arr)
    check(_lib.load().tlx_cumsum(_stream(), _ptr(arr), _ptr(out), arr.shape[0], arr.shape[1], dtype_code(arr),
                                 int(axis), int(bool(reverse))))
    return out


def canonicalize_keys_(x: torch.Tensor) -> torch.Tensor:
    """In place: floats as they look after the key-domain round trip (-0 -> +0, canonical NaN)."""
    x = _dev(x)
    if x.is_floating_point():
        if not x.is_contiguous():
            raise ValueError("canonicalize_keys_ needs a contiguous tensor")
        check(_lib.load().tlx_canonicalize_keys(_stream(), _ptr(x), dtype_code(x), x.numel()))
    return x


def argmax(keys: torch.Tensor, axis: int) -> torch.Tensor:
    keys = _dev(keys)
    out = torch.empty(keys.shape[1 - axis], dtype=torch.int32, device=keys.device)
    check(_lib.load().tlx_argmax(_stream(), _ptr(keys), dtype_code(keys), keys.shape[0], keys.shape[1], int(axis),
                                 _ptr(out)))
    return out


def argsort_rows(keys: torch.Tensor, descending: bool = False, in_perm: torch.Tensor | None = None,
                 want_keys: bool = True, want_perm: bool = True):
    """Stable argsort of every row; returns (sorted_keys | None, perm | None)."""
    keys = _dev(keys)
    rows, n = keys.shape
    lib = _lib.load()
    out_keys = torch.empty_like(keys) if want_keys else None
    out_perm = torch.empty((rows, n), dtype=torch.int32, device=keys.device) if want_perm else None
    nbytes = lib.tlx_sort_workspace_bytes(rows, n)
    ws = _ws(nbytes, keys.device)
    check(lib.tlx_sort(_stream(), _ptr(keys), dtype_code(keys), rows, n, int(bool(descending)), _ptr(in_perm),
                       _ptr(out_keys), _ptr(out_perm), _ptr(ws), ws.numel()))
    return out_keys, out_perm


def top_k(x: torch.Tensor, k_max: int, k_per_row=None, replace_val=None, single_pass: bool = False):
    """Returns (vals, idx) or, with single_pass, (vals, idx, valid, depths, cutoff)."""
    x = _dev(x)
    if x.ndim != 2:
        raise ValueError("Only 2D inputs supported")
    rows, n = x.shape
    dev = x.device
    vals = torch.empty((rows, k_max), dtype=x.dtype, device=dev)
    idx = torch.empty((rows, k_max), dtype=torch.int32, device=dev)
    kpr = _i32vec(k_per_row, rows, dev) if (k_per_row is not None and replace_val is not None) else None
    valid = depths = cutoff = None
    if single_pass:
        valid = torch.empty(1, dtype=torch.int32, device=dev)
        depths = torch.empty(rows, dtype=torch.int32, device=dev)
        cutoff = torch.empty(rows, dtype=torch.int32 if x.dtype == torch.int32 else torch.float32, device=dev)
    lib = _lib.load()
    ws_bytes = 0 if single_pass else lib.tlx_top_k_workspace_bytes(rows, n, int(k_max))   # a few long rows: split over CTAs
    ws = _ws(ws_bytes, dev) if ws_bytes else None
    check(lib.tlx_top_k(_stream(), _ptr(x.contiguous()), dtype_code(x), rows, n, n, int(k_max), _ptr(kpr),
                        int(kpr is not None), float(replace_val if replace_val is not None else 0.0),
                        int(single_pass), _ptr(vals), _ptr(idx), _ptr(valid), _ptr(depths), _ptr(cutoff), _ptr(ws),
                        ws.numel() if ws is not None else 0))
    if single_pass:
        return vals, idx, valid, depths, cutoff
    return vals, idx


def sparse_random_uniform(key, idx0: torch.Tensor, idx1: torch.Tensor, dim1_size: int, minval=0.0, maxval=1.0):
    idx0, idx1 = _dev(idx0).to(torch.int32), _dev(idx1).to(torch.int32)
    if idx0.shape != idx1.shape:
        raise ValueError("index arrays must have the same shape")
    out = torch.empty(idx0.shape, dtype=torch.float32, device=idx0.device)
    kd = key_operand(key)
    if kd is not None:
        check(_lib.load().tlx_sparse_random_uniform_dev(_stream(), _ptr(kd), _ptr(idx0), _ptr(idx1), idx0.numel(),
                                                        int(dim1_size), float(minval), float(maxval), _ptr(out)))
        return out
    k0, k1 = key_pair(key)
    check(_lib.load().tlx_sparse_random_uniform(_stream(), k0, k1, _ptr(idx0), _ptr(idx1), idx0.numel(),
                                                int(dim1_size), float(minval), float(maxval), _ptr(out)))
    return out


def top_p_mask(topk_logits, p, replace_val):
    x = _dev(topk_logits)
    if x.dtype != torch.float32:
        x = x.float()
    k, batch = x.shape
    out = torch.empty_like(x)
    check(_lib.load().tlx_top_p_mask(_stream(), _ptr(x), _ptr(_f32vec(p, batch, x.device)), k, batch,
                                     float(replace_val), _ptr(out)))
    return out


def gumbel_argmax(key, logits, idx0, idx1, dim1_size, axis):
    """Returns [idx0 at winner, idx1 at winner] along `axis` (1-D each)."""
    logits = _dev(logits).float()
    idx0, idx1 = _dev(idx0).to(torch.int32), _dev(idx1).to(torch.int32)
    rows, cols = logits.shape
    pos = torch.empty(rows if axis == 1 else cols, dtype=torch.int32, device=logits.device)
    kd = key_operand(key)
    if kd is not None:
        check(_lib.load().tlx_gumbel_argmax_dev(_stream(), _ptr(logits), _ptr(idx0), _ptr(idx1), rows, cols, _ptr(kd),
                                                int(dim1_size), int(axis), _ptr(pos)))
    else:
        k0, k1 = key_pair(key)
        check(_lib.load().tlx_gumbel_argmax(_stream(), _ptr(logits), _ptr(idx0), _ptr(idx1), rows, cols, k0, k1,
                                            int(dim1_size), int(axis), _ptr(pos)))
    sel = pos.reshape(-1, 1) if axis == 1 else pos.reshape(1, -1)
    return [take_along_axis(i, sel, axis).reshape(-1) for i in (idx0, idx1)]


def top_p_and_sample(topk_logits, topk_idx, top_p, temperature, *, vocab_size, replace_val, rng_key=None, noise=None,
                     dim0_offset=0):
    topk_logits, topk_idx = _dev(topk_logits), _dev(topk_idx).to(torch.int32)
    rows, k = topk_logits.shape
    dev = topk_logits.device
    if noise is not None:
        noise = _dev(noise)
        if noise.dtype != torch.float32 or noise.ndim != 2:
            raise ValueError("noise must be a float32 [batch, vocab] tensor")
    elif rng_key is None:
        raise ValueError("either rng_key or noise is required")
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    kd, od = key_operand(rng_key), offset_operand(dim0_offset)
    if kd is not None or od is not None:
        if kd is None and noise is None:
            kd = torch.tensor(key_pair(rng_key), dtype=torch.int64, device=dev).to(torch.int32)
        check(_lib.load().tlx_top_p_and_sample_dev(
            _stream(), _ptr(topk_logits), dtype_code(topk_logits), _ptr(topk_idx), rows, k,
            _ptr(_f32vec(top_p, rows, dev)), _ptr(_f32vec(temperature, rows, dev)), _ptr(noise),
            noise.shape[1] if noise is not None else 0, _ptr(kd), int(vocab_size), float(replace_val),
            _ptr(od if od is not None else _host_offset(dim0_offset, dev)), _ptr(out)))
        return out
    k0, k1 = key_pair(rng_key)
    check(_lib.load().tlx_top_p_and_sample(
        _stream(), _ptr(topk_logits), dtype_code(topk_logits), _ptr(topk_idx), rows, k, _ptr(_f32vec(top_p, rows, dev)),
        _ptr(_f32vec(temperature, rows, dev)), _ptr(noise), noise.shape[1] if noise is not None else 0, k0, k1,
        int(vocab_size), float(replace_val), int(dim0_offset), _ptr(out)))
    return out


class SampleWorkspace:
    """Reusable buffers for `sample` so that a decode loop does not allocate per step."""

    def __init__(self, rows: int, vocab: int, device):
        lib = _lib.load()
        self.rows, self.vocab = rows, vocab
        self.ws = _ws(lib.tlx_sample_workspace_bytes(rows, vocab), device)
        self.tokens = torch.empty(rows, dtype=torch.int32, device=device)
        self.status = torch.empty(rows, dtype=torch.int32, device=device)


def sample(logits, top_k_, top_p, temperature, *, rng_key=None, noise=None, dim0_offset=0, workspace=None,
           return_status=False):
    """Fused sampler: logits [B, V] -> int32 tokens [B]."""
    logits = _dev(logits)
    if logits.ndim != 2:
        raise ValueError("Only 2D inputs supported")
    rows, vocab = logits.shape
    dev = logits.device
    if noise is not None:
        noise = _dev(noise)
        if noise.dtype != torch.float32 or noise.ndim != 2 or noise.shape[1] < vocab:
            raise ValueError("noise must be a float32 [batch, vocab] tensor")
    elif rng_key is None:
        raise ValueError("either rng_key or noise is required")
    w = workspace if workspace is not None else SampleWorkspace(rows, vocab, dev)
    kd, od = key_operand(rng_key), offset_operand(dim0_offset)
    if kd is not None or od is not None:
        # key and/or offset live on the device: they are handed over as device operands
        if kd is None and noise is None:
            kd = torch.tensor(key_pair(rng_key), dtype=torch.int64, device=dev).to(torch.int32)
        check(_lib.load().tlx_sample_dev(
            _stream(), _ptr(logits), dtype_code(logits), rows, vocab, vocab, _ptr(_i32vec(top_k_, rows, dev)),
            _ptr(_f32vec(top_p, rows, dev)), _ptr(_f32vec(temperature, rows, dev)), _ptr(noise),
            noise.shape[1] if noise is not None else 0, _ptr(kd),
            _ptr(od if od is not None else _host_offset(dim0_offset, dev)), _ptr(w.tokens), _ptr(w.status),
            _ptr(w.ws), w.ws.numel()))
        return (w.tokens, w.status) if return_status else w.tokens
    k0, k1 = key_pair(rng_key)
    check(_lib.load().tlx_sample(
        _stream(), _ptr(logits), dtype_code(logits), rows, vocab, vocab, _ptr(_i32vec(top_k_, rows, dev)),
        _ptr(_f32vec(top_p, rows, dev)), _ptr(_f32vec(temperature, rows, dev)), _ptr(noise),
        noise.shape[1] if noise is not None else 0, k0, k1, int(dim0_offset), _ptr(w.tokens), _ptr(w.status),
        _ptr(w.ws), w.ws.numel()))
    if return_status:
        return w.tokens, w.status
    return w.tokens


def shard_candidates(logits_shard, col_offset: int, k_cand: int, *, noise_shard=None, rng_key=None, vocab_total=None,
                     dim0_offset=0, out=None):
    """One vocab shard's local top-k' as a packed float32/int32 block [3, rows, k'] (values, global token ids
    bit-cast to float32 storage, noise) ready for an all-gather."""
    logits_shard = _dev(logits_shard)
    rows, v_local = logits_shard.shape
    dev = logits_shard.device
    if noise_shard is not None:
        noise_shard = _dev(noise_shard)
    elif rng_key is None:
        raise ValueError("either rng_key or noise_shard is required")
    if out is None:
        out = torch.empty((3, rows, k_cand), dtype=torch.float32, device=dev)
    kd, od = key_operand(rng_key), offset_operand(dim0_offset)
    if kd is not None or od is not None:
        if kd is None and noise_shard is None:
            kd = torch.tensor(key_pair(rng_key), dtype=torch.int64, device=dev).to(torch.int32)
        check(_lib.load().tlx_shard_candidates_dev(
            _stream(), _ptr(logits_shard), dtype_code(logits_shard), rows, v_local, v_local, int(col_offset),
            int(k_cand), _ptr(noise_shard), noise_shard.shape[1] if noise_shard is not None else 0, _ptr(kd),
            int(vocab_total if vocab_total is not None else v_local),
            _ptr(od if od is not None else _host_offset(dim0_offset, dev)), out[0].data_ptr(), out[1].data_ptr(),
            out[2].data_ptr(), None, 0))
        return out
    k0, k1 = key_pair(rng_key)
    check(_lib.load().tlx_shard_candidates(
        _stream(), _ptr(logits_shard), dtype_code(logits_shard), rows, v_local, v_local, int(col_offset), int(k_cand),
        _ptr(noise_shard), noise_shard.shape[1] if noise_shard is not None else 0, k0, k1,
        int(vocab_total if vocab_total is not None else v_local), int(dim0_offset), out[0].data_ptr(),
        out[1].data_ptr(), out[2].data_ptr(), None, 0))
    return out


def merge_and_sample(gathered, top_k_, top_p, temperature, out=None):
    """gathered: [n_shards, 3, rows, k'] float32 storage as produced by all-gathering `shard_candidates` blocks."""
    gathered = _dev(gathered)
    n_shards, three, rows, k = gathered.shape
    assert three == 3
    dev = gathered.device
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=dev)
    block = 3 * rows * k
    check(_lib.load().tlx_merge_and_sample(
        _stream(), gathered[0, 0].data_ptr(), gathered[0, 1].data_ptr(), gathered[0, 2].data_ptr(), rows,
        n_shards * k, k, block, k, _ptr(_i32vec(top_k_, rows, dev)), _ptr(_f32vec(top_p, rows, dev)),
        _ptr(_f32vec(temperature, rows, dev)), _ptr(out)))
    return out


# ---- vocab-sharded sampler with the candidates exchanged over peer memory ------------------------------
class Exchange:
    """This rank's exchange buffer and the other ranks' buffers as mapped here (C ABI: tlx_exchange_*).

    `Exchange.create(rows, k_cand, world)` allocates the local buffer and returns it with its 64-byte
    inter-process handle; `attach(rank, handles)` maps the other ranks' buffers from their handles.
    `Exchange.local_group(rows, k_cand, world)` makes `world` buffers in this process (several ranks stood
    in for by one device, or one process driving several devices)."""

    def __init__(self, rows, k_cand, world):
        self.rows, self.k_cand, self.world = int(rows), int(k_cand), int(world)
        self.rank = None
        self.own = None          # device address of this rank's buffer
        self.handle = None
        self.peers = None        # ctypes array of `world` device addresses
        self._opened = []
        self.status = None

    @classmethod
    def create(cls, rows, k_cand, world, device=None):
        import ctypes
        self = cls(rows, k_cand, world)
        buf = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(dev):
            check(_lib.load().tlx_exchange_create(self.rows, self.k_cand, self.world, ctypes.byref(buf), handle))
            self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.device = dev
        self.own = buf.value
        self.handle = bytes(handle)
        return self

    def attach(self, rank, handles):
        """handles: the `world` ranks' handles in rank order (this rank's own entry is not opened)."""
        import ctypes
        assert len(handles) == self.world
        self.rank = int(rank)
        ptrs = []
        with torch.cuda.device(self.device):
            for i, h in enumerate(handles):
                if i == self.rank:
                    ptrs.append(self.own)
                    continue
                peer = ctypes.c_void_p()
                hb = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                check(_lib.load().tlx_exchange_open(hb, ctypes.byref(peer)))
                self._opened.append(peer.value)
                ptrs.append(peer.value)
        self.peers = (ctypes.c_void_p * self.world)(*ptrs)
        return self

    @classmethod
    def local_group(cls, rows, k_cand, world, device=None):
        import ctypes
        group = [cls.create(rows, k_cand, world, device) for _ in range(world)]
        for r, e in enumerate(group):
            e.rank = r
            e.peers = (ctypes.c_void_p * world)(*[g.own for g in group])
        return group

    def state(self):
        """(steps completed, error word) of this rank's buffer; synchronises the current stream."""
        import ctypes
        steps, err = ctypes.c_uint32(), ctypes.c_uint32()
        check(_lib.load().tlx_exchange_status(_stream(), self.own, ctypes.byref(steps), ctypes.byref(err)))
        return steps.value, err.value

    def close(self):
        """Unmaps the other ranks' buffers and frees this rank's own (no rank may still write to it)."""
        lib = _lib.load()
        for p in self._opened:
            lib.tlx_exchange_close(p)
        self._opened = []
        if self.own:
            lib.tlx_exchange_destroy(self.own)
            self.own = None

    def __del__(self):
        try:
            self.close()
        except Exception:      # interpreter shutdown: the library or the CUDA context may be gone already
            pass


def exchange_shard_candidates(logits_shard, col_offset: int, exchange: Exchange, *, noise_shard=None, rng_key=None,
                              vocab_total=None, dim0_offset=0):
    """Stage 1 with the exchange fused in: this rank's top-k' of every row goes straight into every rank's
    exchange buffer."""
    logits_shard = _dev(logits_shard)
    rows, v_local = logits_shard.shape
    dev = logits_shard.device
    if (rows, ) != (exchange.rows, ):
        raise ValueError("exchange was made for another row count")
    if noise_shard is not None:
        noise_shard = _dev(noise_shard)
    elif rng_key is None:
        raise ValueError("either rng_key or noise_shard is required")
    kd, od = key_operand(rng_key), offset_operand(dim0_offset)
    k0 = k1 = 0
    if kd is None and noise_shard is None:
        k0, k1 = key_pair(rng_key)
    check(_lib.load().tlx_exchange_shard_candidates(
        _stream(), _ptr(logits_shard), dtype_code(logits_shard), rows, v_local, v_local, int(col_offset),
        exchange.k_cand, _ptr(noise_shard), noise_shard.shape[1] if noise_shard is not None else 0, _ptr(kd), k0, k1,
        int(vocab_total if vocab_total is not None else v_local), 0 if od is not None else int(dim0_offset), _ptr(od),
        exchange.rank, exchange.world, exchange.peers))


def exchange_merge_and_sample(exchange: Exchange, top_k_, top_p, temperature, out=None):
    """Stage 2 on this rank's exchange buffer: waits per row for all ranks' candidates, merges, samples."""
    rows = exchange.rows
    dev = exchange.device
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=dev)
    check(_lib.load().tlx_exchange_merge_and_sample(
        _stream(), exchange.own, rows, exchange.k_cand, exchange.world, _ptr(_i32vec(top_k_, rows, dev)),
        _ptr(_f32vec(top_p, rows, dev)), _ptr(_f32vec(temperature, rows, dev)), _ptr(out), _ptr(exchange.status)))
    return out
