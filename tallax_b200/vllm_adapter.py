"""vLLM-convention front end of the fused sampler.

`tallax/_src/sampling.py:331-341` reads `.top_k`, `.top_p` and `.temperature` from the metadata object
vLLM's TPU runner hands it.  vLLM's own conventions are wider than what that code (and the kernel behind
`tallax_b200.sampling.sample`) accepts; this module maps them:

  * `top_k = -1` (vLLM's "disabled"), 0, or >= vocab  ->  0 (the kernel's "disabled");
  * `top_p` missing -> 1.0; `temperature` missing -> 1.0; `temperature = 0` is greedy (the kernel treats
    every temperature below 1e-5 as greedy, as the reference does);
  * `min_p`: a token survives if softmax(x / T)_i >= min_p * max_j softmax(x / T)_j, which is the value test
    x_i >= max(x) + T * log(min_p).  The kernel has no such operand: rows with min_p > 0 get their logits
    below that value set to -inf before the call (one extra pass over those rows, through this library's
    arg-max kernel for the row maxima; rows without min_p are not touched);
  * per-request seeds: a seeded request must draw the same noise wherever it sits in the batch, so each
    seeded row is sampled in a call of its own with a key derived from (seed, step) and row offset 0; the
    unseeded rows share the step's key in one call.

Not mapped: penalties and logit bias act on the logits before sampling and belong to the caller.
Semantics stay the reference's where the two differ: the top-p mass is taken over the softmax of the
UNSCALED logits (sampling.py:45-46) and the temperature divides afterwards (sampling.py:97), whereas vLLM's
GPU sampler scales first.  `scale_before_top_p=True` gives vLLM's order (the logits are divided by the
temperature up front, one extra pass, and the kernel runs at temperature 1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Optional, Sequence

import torch

_GREEDY_EPS = 1e-5


@dataclass
class VllmSamplingParams:
    """Per-request vectors in vLLM's conventions (tensors or sequences of length batch; None = default)."""
    temperature: Any = None
    top_k: Any = None
    top_p: Any = None
    min_p: Any = None
    seeds: Optional[Sequence[Optional[int]]] = None   # per request; None = unseeded


def normalize_top_k(top_k, batch: int, vocab: int, device=None) -> torch.Tensor:
    """vLLM's top_k (-1 or 0 = disabled, otherwise a count) as the kernel's int32 vector (0 = disabled)."""
    if top_k is None:
        return torch.zeros(batch, dtype=torch.int32, device=device)
    t = torch.as_tensor(top_k, device=device).to(torch.int64).reshape(-1)
    if t.numel() == 1:
        t = t.expand(batch)
    if t.numel() != batch:
        raise ValueError("top_k must have one entry per request")
    if bool((t < -1).any()):
        raise ValueError("top_k must be -1 (disabled) or >= 0")
    return torch.where((t <= 0) | (t >= vocab), torch.zeros_like(t), t).to(torch.int32)


def _vector(v, default: float, batch: int, device) -> torch.Tensor:
    if v is None:
        return torch.full((batch,), default, dtype=torch.float32, device=device)
    t = torch.as_tensor(v, device=device).to(torch.float32).reshape(-1)
    if t.numel() == 1:
        t = t.expand(batch).contiguous()
    if t.numel() != batch:
        raise ValueError("per-request vectors must have one entry per request")
    return t


def min_p_threshold(row_max: torch.Tensor, temperature: torch.Tensor, min_p: torch.Tensor) -> torch.Tensor:
    """Smallest logit that survives min_p: max + T * log(min_p); -inf where min_p is 0 (nothing is cut) and
    for greedy rows."""
    safe = torch.clamp(min_p, min=1e-38)
    thr = row_max.to(torch.float32) + temperature * torch.log(safe)
    off = (min_p <= 0) | (temperature < _GREEDY_EPS)
    return torch.where(off, torch.full_like(thr, -math.inf), thr)


def request_key(seed: int, step: int) -> tuple[int, int]:
    """Threefry key of a seeded request at a decode step: the seed's two 32-bit halves, the step mixed into
    the high word (an odd multiplier, so that different steps give different keys for every seed)."""
    seed &= (1 << 64) - 1
    lo, hi = seed & 0xFFFFFFFF, seed >> 32
    return lo, (hi ^ ((step * 0x9E3779B1) & 0xFFFFFFFF)) & 0xFFFFFFFF


def _row_max(logits: torch.Tensor) -> torch.Tensor:
    from tallax_b200._src import ops
    idx = ops.argmax(logits, axis=1)
    return logits.gather(1, idx.reshape(-1, 1).to(torch.int64)).reshape(-1)


def sample(step_key, logits: torch.Tensor, params: VllmSamplingParams, *, step: int = 0,
           scale_before_top_p: bool = False, sample_fn: Optional[Callable] = None,
           row_max_fn: Optional[Callable] = None) -> torch.Tensor:
    """Token ids int32 [batch] for logits [batch, vocab] under vLLM-convention parameters.

    step_key: the decode step's threefry key (two 32-bit words) for the unseeded requests.
    sample_fn / row_max_fn: the sampler and the row-maximum routine; default to this library's
    (`tallax_b200.sampling.sample`, its arg-max kernel).  Tests pass CPU stand-ins.
    """
    from tallax_b200._src.sampling import SamplingMetadata
    if sample_fn is None:
        from tallax_b200._src.sampling import sample as sample_fn
    if row_max_fn is None:
        row_max_fn = _row_max
    if logits.ndim != 2:
        raise ValueError("Only 2D inputs supported")
    batch, vocab = logits.shape
    dev = logits.device
    top_k = normalize_top_k(params.top_k, batch, vocab, dev)
    top_p = _vector(params.top_p, 1.0, batch, dev)
    temperature = _vector(params.temperature, 1.0, batch, dev)
    if bool(((top_p <= 0) | (top_p > 1)).any()):
        raise ValueError("top_p must be in (0, 1]")
    if bool((temperature < 0).any()):
        raise ValueError("temperature must be >= 0")
    min_p = _vector(params.min_p, 0.0, batch, dev)
    if bool(((min_p < 0) | (min_p > 1)).any()):
        raise ValueError("min_p must be in [0, 1]")

    x = logits
    if scale_before_top_p:
        live = temperature >= _GREEDY_EPS
        scale = torch.where(live, 1.0 / torch.clamp(temperature, min=_GREEDY_EPS), torch.ones_like(temperature))
        x = (logits.to(torch.float32) * scale[:, None]).to(logits.dtype)
        min_temperature = torch.ones_like(temperature)          # min_p now acts on the scaled logits
        temperature = torch.where(live, torch.ones_like(temperature), temperature)
    else:
        min_temperature = temperature
    rows_min_p = torch.nonzero(min_p > 0).flatten()
    if rows_min_p.numel():
        sub = x[rows_min_p]
        thr = min_p_threshold(row_max_fn(sub), min_temperature[rows_min_p], min_p[rows_min_p])
        sub = torch.where(sub.to(torch.float32) < thr[:, None], torch.full_like(sub, -math.inf), sub)
        x = x.clone() if x is logits else x
        x[rows_min_p] = sub

    seeds = list(params.seeds) if params.seeds is not None else [None] * batch
    if len(seeds) != batch:
        raise ValueError("seeds must have one entry per request")
    seeded = [i for i, s in enumerate(seeds) if s is not None]
    out = torch.empty(batch, dtype=torch.int32, device=dev)
    unseeded = [i for i in range(batch) if seeds[i] is None]
    if unseeded:
        if len(unseeded) == batch:
            md = SamplingMetadata(top_k=top_k, top_p=top_p, temperature=temperature)
            out.copy_(sample_fn(step_key, x, md))
        else:
            sel = torch.tensor(unseeded, device=dev)
            md = SamplingMetadata(top_k=top_k[sel], top_p=top_p[sel], temperature=temperature[sel])
            out[sel] = sample_fn(step_key, x[sel].contiguous(), md).to(torch.int32)
    for i in seeded:
        md = SamplingMetadata(top_k=top_k[i:i + 1], top_p=top_p[i:i + 1], temperature=temperature[i:i + 1])
        out[i:i + 1] = sample_fn(request_key(int(seeds[i]), step), x[i:i + 1].contiguous(), md).to(torch.int32)
    return out
