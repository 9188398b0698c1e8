#!/usr/bin/env python
"""Benchmark of the fused decode sampler: bf16 logits [256, 128256] per GPU -> token ids.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one fused-sampler call over one batch (256 rows per GPU, weak scaling:
batch rows are independent, each rank samples its own batch, no collective on the data
path).  Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of
the reference's algorithm on the host cores instead (rank 0 only), on the 256 rows of the
same input set 0 that the GPU arm's first step reads.

Side records in the same line: `replay_200` (200 further graph launches, a steadier mean),
`e2e_key_noise` (end to end with threefry noise from a key instead of an uploaded noise
tensor), and with more than one GPU `strong` (the 256 rows split over the ranks,
dim0_offset = rank * 256 / N) and `vocab_sharded` (benchmark configuration 5: the vocabulary
split over the ranks, NCCL all-gather of the candidates).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, V = 256, 128256          # benchmark configuration: decode batch and vocabulary (Llama-3 sized)
N_SETS = 4                  # rotating input sets: 4 x 65.7 MB of logits > 126 MB L2, so every step reads HBM
ALGO_BYTES = B * V * 2 + B * 12 + B * 4   # logits once + three parameter vectors + tokens out
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ncu_dram_traffic_sample_c3.json")   # from one ncu capture
METRIC, UNIT = "sampled_tokens_per_s", "tokens/s"
WORKLOAD = ("fused temperature/top-k/top-p/noise sampling, bf16 logits [256,128256] = N(0,sigma=3) + 10 at 8 "
            "columns per row, T~U[0.5,1.5], top_k~U{1..1024} with 10% disabled, top_p~U[0.6,1), explicit f32 "
            "uniform noise [256,128256]")


def bench_config(rows_call, world):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "batch_per_gpu": rows_call, "vocab": V, "sharding": f"batch rows x{world}",
            "l2": f"{N_SETS} rotating input sets ({N_SETS * rows_call * V * 6 / 1e6:.0f} MB of logits and noise > 126 MB "
                  "L2)"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def ncu_traffic():
    """dram bytes read + written by the kernels of one sampler call, from the committed summary of an ncu
    capture of this workload (None if the file is missing)."""
    try:
        with open(TRAFFIC_FILE) as f:
            return int(json.load(f)["dram_bytes_per_call"])
    except Exception:
        return None


def make_inputs_host(seed, rows=B):
    """One synthetic input set with the configuration's shapes and distributions, as NumPy arrays (Philox
    stream `seed`).  Both arms draw their inputs here, so that they sample the same rows."""
    import ml_dtypes
    import numpy as np
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.standard_normal((rows, V), dtype=np.float32) * np.float32(3.0)
    cols = np.argsort(rng.random((rows, 64), dtype=np.float32), axis=1)[:, :8] * (V // 64) + rng.integers(0, V // 64, (rows, 8))
    np.add.at(x, (np.arange(rows)[:, None], cols), np.float32(10.0))
    temperature = rng.uniform(0.5, 1.5, size=rows).astype(np.float32)
    top_k = rng.integers(1, 1025, size=rows).astype(np.int32)
    top_k[rng.random(rows) < 0.1] = 0
    top_p = rng.uniform(0.6, 1.0, size=rows).astype(np.float32)
    noise = rng.random((rows, V), dtype=np.float32)
    return x.astype(ml_dtypes.bfloat16), top_k, top_p, temperature, noise


def make_inputs(torch, device, seed, rows=B):
    """The same input set on the device."""
    x, top_k, top_p, temperature, noise = make_inputs_host(seed, rows)
    logits = torch.from_numpy(x.view("int16")).view(torch.bfloat16).to(device)
    return (logits, torch.from_numpy(top_k).to(device), torch.from_numpy(top_p).to(device),
            torch.from_numpy(temperature).to(device), torch.from_numpy(noise).to(device))


def to_numpy(t):
    import torch
    if t.dtype == torch.bfloat16:
        import ml_dtypes
        return t.cpu().view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.cpu().numpy()


_REF_DATA = None


def _oracle_rows(i):
    from oracle import tallax_oracle as o
    x, tk, tp, T, noise, stride = _REF_DATA
    return o.sample(x[i::stride], tk[i::stride], tp[i::stride], T[i::stride], noise=noise[i::stride])


def run_reference(args):
    """CPU arm: the NumPy restatement of the reference's algorithm, rows spread over all host cores."""
    global _REF_DATA
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import multiprocessing as mp
    from oracle import tallax_oracle as o
    cores = os.cpu_count() or 1
    # all 256 rows of input set 0 (the set the GPU arm's first step reads); with few host cores a bounded
    # sample of its first rows, so that the run still ends within minutes
    rows = B if cores >= 16 else max(cores, 8) * 4
    workers = min(cores, rows)
    _REF_DATA = (*(a[:rows] for a in make_inputs_host(0)), workers)
    chunks = list(range(workers))
    with mp.get_context("fork").Pool(workers) as pool:  # forked after the data exists: workers inherit it
        for _ in range(args.warmup):
            pool.map(_oracle_rows, chunks)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            pool.map(_oracle_rows, chunks)
        dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(B, int(os.environ.get("WORLD_SIZE", "1"))),   # the GPU arm's config, key for key
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": len(chunks), "kind": "port",
                         "sample": f"{'all' if rows == B else 'the first'} {rows} of the 256 rows of input set 0 per "
                                   "step, NumPy restatement (JAX is not installable here)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from tallax_b200 import _lib, sampling
    from tallax_b200._src import ops
    _lib.load()

    rows_call = args.rows_per_call or B   # 32 / 64 / 128: the same rows in smaller calls (a smaller decode batch)
    sets = [make_inputs(torch, device, seed=1000 * rank + s, rows=rows_call) for s in range(N_SETS)]
    if args.mix != "c3":
        # the same logits and noise with another mix of sampling parameters (kernel time only, one GPU)
        def remix(s):
            x, tk, tp, T, u = s
            if args.mix == "greedy":
                T = torch.zeros_like(T)
            elif args.mix in ("k1", "k50", "k1024"):
                tk = torch.full_like(tk, int(args.mix[1:]))
            elif args.mix == "no-wide":
                tk = torch.where(tk == 0, torch.full_like(tk, 500), tk)
            elif args.mix == "all-wide":
                tk = torch.zeros_like(tk)
            return (x, tk, tp, T, u)
        sets = [remix(s) for s in sets]
    ws = ops.SampleWorkspace(rows_call, V, device)
    meta = [sampling.SamplingMetadata(top_k=s[1], top_p=s[2], temperature=s[3]) for s in sets]

    def step(i):
        s = sets[i % N_SETS]
        return sampling.sample(None, s[0], meta[i % N_SETS], noise=s[4], workspace=ws)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib = _lib.load()
    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    # One CUDA graph per input set, each holding one sampler call: a timed step is one graph launch, so
    # that the host's launch path (Python, ctypes, several driver calls per step) is not what is measured.
    graphs, launches_per_call = [], 0
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for j in range(N_SETS):
                g = torch.cuda.CUDAGraph()
                before = lib.tlx_kernel_launches()
                with torch.cuda.graph(g, stream=side):
                    step(j)
                launches_per_call = lib.tlx_kernel_launches() - before
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        for j in range(N_SETS):
            graphs[j].replay()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        time.sleep(0.15)
        barrier()
        launches0 = lib.tlx_kernel_launches()
        start.record()
        for i in range(args.steps):
            if graphs:
                graphs[i % N_SETS].replay()
            else:
                step(i)
        stop.record()
        launches = (launches_per_call * args.steps) if graphs else (lib.tlx_kernel_launches() - launches0)
        barrier()
        time.sleep(0.1)
    ms = start.elapsed_time(stop)
    rank_ms = ms
    # a steadier mean: 200 further graph launches
    replay_ms = None
    if graphs:
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        r0.record()
        for i in range(200):
            graphs[i % N_SETS].replay()
        r1.record()
        barrier()
        replay_ms = r0.elapsed_time(r1) / 200

    if args.mix != "c3":
        if rank == 0:
            per_step = ms / args.steps
            peak, peak_src = peaks()
            algo = rows_call * V * 2 + rows_call * 16
            print(json.dumps({
                "metric": METRIC, "value": rows_call / (per_step / 1e3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": dict(bench_config(rows_call, 1), mix=args.mix),
                "clocks": clocks.summary(), "gpu_launches": int(launches),
                "replay_200": {"ms_per_step": replay_ms},
                "roofline": {"bound": "hbm", "achieved": algo / (per_step / 1e3) / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": algo / (per_step / 1e3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                             "note": "logits once + parameters + tokens; kernel time only, no end-to-end or CPU leg"}}),
                  flush=True)
        return

    # ---- end to end through the public API from pinned host buffers --------------------------
    h_logits = torch.empty((rows_call, V), dtype=torch.bfloat16).pin_memory()
    h_noise = torch.empty((rows_call, V), dtype=torch.float32).pin_memory()
    h_params = [torch.empty(rows_call, dtype=t.dtype).pin_memory() for t in sets[0][1:4]]
    h_logits.copy_(sets[0][0]); h_noise.copy_(sets[0][4])
    for h, t in zip(h_params, sets[0][1:4]):
        h.copy_(t)
    d_logits, d_noise = torch.empty_like(sets[0][0]), torch.empty_like(sets[0][4])
    d_params = [torch.empty_like(t) for t in sets[0][1:4]]
    h_tokens = torch.empty(rows_call, dtype=torch.int32).pin_memory()
    key = (0x243F6A88, 0x85A308D3)

    def e2e_step(with_noise=True):
        d_logits.copy_(h_logits, non_blocking=True)
        if with_noise:
            d_noise.copy_(h_noise, non_blocking=True)
        for d, h in zip(d_params, h_params):
            d.copy_(h, non_blocking=True)
        md = sampling.SamplingMetadata(top_k=d_params[0], top_p=d_params[1], temperature=d_params[2])
        if with_noise:
            tok = sampling.sample(None, d_logits, md, noise=d_noise, workspace=ws)
        else:   # the reference's own calling convention: a PRNG key, the noise is generated where it is needed
            tok = sampling.sample(key, d_logits, md, workspace=ws)
        h_tokens.copy_(tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller needs the token ids before the next decode step

    e2e_steps = max(3, min(args.steps, 20))

    def time_e2e(with_noise):
        for _ in range(2):
            e2e_step(with_noise)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step(with_noise)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    e2e_ms = time_e2e(True)
    e2e_key_ms = time_e2e(False)

    # ---- the 256 rows split over the ranks (strong scaling): rank r samples rows [r*B/N, (r+1)*B/N) of ONE
    # global batch, its noise counters offset by dim0_offset = r*B/N, as the reference's batch sharding does
    strong_ms, strong_mismatches = None, None
    if world > 1 and B % world == 0 and not args.rows_per_call:
        bl = B // world
        g_sets = [make_inputs(torch, device, seed=5000 + s) for s in range(N_SETS)]   # the same on every rank
        s_sets = [tuple(t[rank * bl:(rank + 1) * bl].contiguous() for t in gs[:4]) for gs in g_sets]
        g0 = g_sets[0][:4]
        del g_sets
        s_ws = ops.SampleWorkspace(bl, V, device)
        s_meta = [sampling.SamplingMetadata(top_k=t[1], top_p=t[2], temperature=t[3]) for t in s_sets]

        def strong_step(i):
            return sampling.sample(key, s_sets[i % N_SETS][0], s_meta[i % N_SETS], workspace=s_ws,
                                   dim0_offset=rank * bl)

        # parity: the ranks' tokens, side by side, are the tokens of the unsharded call with the same key
        mine = strong_step(0).clone()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        if rank == 0:
            whole = sampling.sample(key, g0[0], sampling.SamplingMetadata(top_k=g0[1], top_p=g0[2], temperature=g0[3]))
            strong_mismatches = int((torch.cat(parts) != whole).sum())
        del g0
        for i in range(4):
            strong_step(i)
        barrier()
        s_graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for j in range(N_SETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    strong_step(j)
                s_graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        for g in s_graphs:
            g.replay()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for i in range(100):
            s_graphs[i % N_SETS].replay()
        s1.record()
        barrier()
        strong_ms = s0.elapsed_time(s1) / 100

    # ---- benchmark configuration 5 on the same ranks: the vocabulary split, one all-gather of candidates
    vs = vocab_sharded_record(args, torch, dist, device, rank, world) if world > 1 and not args.rows_per_call else None

    times = torch.tensor([ms, e2e_ms, e2e_key_ms, strong_ms or 0.0, replay_ms or 0.0], dtype=torch.float64, device=device)
    per_rank = [rank_ms]
    if world > 1:
        gathered = [torch.zeros(1, dtype=torch.float64, device=device) for _ in range(world)]
        dist.all_gather(gathered, times[:1].clone())
        per_rank = [float(t.item()) for t in gathered]
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_key_ms, strong_ms, replay_ms = times.tolist()

    if rank == 0:
        peak, peak_src = peaks()
        per_step_s = ms / 1e3 / args.steps
        # CPU baseline on a bounded sample of the same workload (rank 0, one core), also a parity spot check
        from oracle import tallax_oracle as o
        # one GPU: all rows of input set 0, repeated until ten seconds of CPU work are done; more GPUs: the
        # first 48 rows once (the baseline is reported at N = 1, the parity check stays)
        n_cpu = rows_call if world == 1 else min(48, rows_call)
        s0 = sets[0]
        xs, tk, tp, T = (to_numpy(t[:n_cpu]) for t in s0[:4])
        nz = to_numpy(s0[4][:n_cpu])
        cpu_reps, cpu_dt = 0, 0.0
        while cpu_reps == 0 or (world == 1 and cpu_dt < 10.0 and cpu_reps < 32):
            t0 = time.perf_counter()
            exp, flags = o.sample(xs, tk, tp, T, noise=nz, return_flags=True)
            cpu_dt += time.perf_counter() - t0
            cpu_reps += 1
        got = to_numpy(sampling.sample(None, s0[0], meta[0], noise=s0[4])[:n_cpu])
        mismatches = int(((got != exp) & ~flags).sum())
        launches_call = launches // max(args.steps, 1)
        algo = ALGO_BYTES * rows_call // B
        achieved = algo / per_step_s / 1e9
        traffic = ncu_traffic() if rows_call == B else None
        line = {
            "metric": METRIC, "value": world * rows_call * args.steps / (ms / 1e3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(rows_call, world),
            "clocks": clocks.summary(),
            "ms_per_step_by_rank": [t / args.steps for t in per_rank],
            "launch": "one CUDA graph launch per step" if graphs else "one library call per step",
            "e2e": {"value": world * rows_call * e2e_steps / (e2e_ms / 1e3), "unit": UNIT,
                    "h2d_bytes_per_step": rows_call * V * 2 + rows_call * V * 4 + rows_call * 12,
                    "d2h_bytes_per_step": rows_call * 4, "ms_per_step": e2e_ms / e2e_steps},
            "e2e_key_noise": {"value": world * rows_call * e2e_steps / (e2e_key_ms / 1e3), "unit": UNIT,
                              "h2d_bytes_per_step": rows_call * V * 2 + rows_call * 12, "d2h_bytes_per_step": rows_call * 4,
                              "ms_per_step": e2e_key_ms / e2e_steps,
                              "note": "the reference's calling convention: a PRNG key instead of an uploaded noise "
                                      "tensor (threefry noise generated on the device)"},
            "gpu_launches": int(launches),
            "replay_200": None if not replay_ms else {"ms_per_step": replay_ms,
                                                      "value": world * rows_call / (replay_ms / 1e3), "unit": UNIT},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_src,
                         "note": "algorithmic bytes of one sampler call (logits once, parameters, tokens) / mean "
                                 f"duration of the whole call (its {launches_call} kernels: prologue, stream, finish), "
                                 "CUDA events on the launching stream; the stream kernel is the dominant one and the "
                                 "only one that reads the logits in full; traffic = dram read+write of the call's "
                                 "kernels, from profiles/ncu_dram_traffic_sample_c3.json (one ncu capture of this "
                                 "workload; it includes the noise of the rows without top-k, which the algorithmic "
                                 "bytes leave out)"},
            "cpu_baseline": {"value": n_cpu * cpu_reps / cpu_dt, "unit": UNIT, "cores": 1, "kind": "port",
                             "sample": f"the first {n_cpu} rows of input set 0, {cpu_reps} time(s) ({cpu_dt:.1f} s of "
                                       f"CPU work), NumPy restatement of the reference (JAX not installable here); "
                                       f"{mismatches} token mismatches vs the GPU outside the 1e-6 top-p exemption"},
        }
        if strong_ms:
            line["strong"] = {"rows_per_gpu": B // world, "ms_per_step": strong_ms, "value": B / (strong_ms / 1e3),
                              "unit": UNIT, "scaling": "strong", "steps": 100, "mismatches": strong_mismatches,
                              "note": "one global batch of 256 rows split over the ranks, dim0_offset = rank * rows_per_gpu, "
                                      "threefry noise from one key; max over ranks"}
        if vs:
            line["vocab_sharded"] = vs
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_op_workload(args):
    """Rows/s and roofline fraction of the other operators at their benchmark sizes (one GPU)."""
    import torch
    from tallax_b200 import _lib, tax, tumpy
    _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev)
    w = args.workload
    if w == "c1":      # exact top-k, f32 [8, 32768], k = 64
        rows, n = 8, 32768
        g.manual_seed(0)
        xs = [torch.randn((rows, n), generator=g, device=dev) for _ in range(4)]
        fn = lambda i: tax.top_k(xs[i % 4], 64)
        algo, note = rows * n * 4 + rows * 64 * 8, "read keys once + write k values and indices"
    elif w == "c2":    # stable ascending sort with payload, f32 [128, 65536]
        rows, n = 128, 65536
        g.manual_seed(1)
        ks = [torch.randn((rows, n), generator=g, device=dev) for _ in range(3)]
        pay = torch.arange(n, dtype=torch.int32, device=dev).repeat(rows, 1)
        fn = lambda i: tax.sort([ks[i % 3], pay], num_keys=1, is_stable=True)
        algo, note = 2 * rows * n * 8, "one read + one write of keys and payload (the op is compare-exchange-bound)"
    elif w in ("c4a", "c4a-single-pass"):   # top-k, f32 [1024, 262144], k = 128
        rows, n = 1024, 262144
        g.manual_seed(3)
        x = torch.randn((rows, n), generator=g, device=dev)   # 1 GiB > L2
        from tallax_b200._src import ops
        fn = (lambda i: tax.top_k(x, 128)) if w == "c4a" else (lambda i: ops.top_k(x, 128, single_pass=True))
        algo, note = rows * n * 4 + rows * 128 * 8, "read keys once + write k values and indices"
    elif w == "c4b":   # gather, i32 indices [1024, 4096] into f32 [1024, 262144]
        rows, n = 1024, 262144
        g.manual_seed(3)
        x = torch.randn((rows, n), generator=g, device=dev)
        ind = torch.randint(0, n, (rows, 4096), generator=g, device=dev, dtype=torch.int32)
        fn = lambda i: tumpy.take_along_axis(x, ind, axis=1)
        algo, note = 3 * rows * 4096 * 4, "indices + gathered elements + output (32-byte sectors: 134 217 728 B)"
    elif w in ("c5-shard-of-8", "c5-merge-of-8"):
        # what ONE rank of an 8-way vocabulary split does per step, on one GPU: the candidate stage on its
        # bf16 [rows, 18992] shard, or the merge of 8 ranks' candidate blocks (k' = 50 each) and the tail.
        # rows = 1024 is configuration 5; --rows scales it (4096 rows make the shard larger than L2).
        from tallax_b200._src import ops
        rows, n, k = (args.rows or 1024), 151936 // 8, 50
        g.manual_seed(4)
        nz = torch.rand((rows, n), generator=g, device=dev)
        shards = [(torch.randn((rows, n), generator=g, device=dev) * 2).to(torch.bfloat16) for _ in range(8)]
        gathered = torch.empty((8, 3, rows, k), dtype=torch.float32, device=dev)
        for r in range(8):
            ops.shard_candidates(shards[r], r * n, k, noise_shard=nz, out=gathered[r])
        blk = torch.empty((3, rows, k), dtype=torch.float32, device=dev)
        tok = torch.empty(rows, dtype=torch.int32, device=dev)
        tk = torch.full((rows,), k, dtype=torch.int32, device=dev)
        tp = torch.full((rows,), 0.95, device=dev)
        T = torch.full((rows,), 0.8, device=dev)
        if w == "c5-shard-of-8":
            fn = lambda i: ops.shard_candidates(shards[i % 8], 0, k, noise_shard=nz, out=blk)
            algo, note = rows * n * 2 + rows * k * 12, "the shard once + its candidates out"
        else:
            fn = lambda i: ops.merge_and_sample(gathered, tk, tp, T, out=tok)
            algo, note = 8 * rows * k * 12 + rows * 4, "8 candidate blocks once + the tokens (latency-bound: 0.6 KB per row and rank)"
    else:
        raise SystemExit(f"unknown workload {w}")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2
    for i in range(max(args.warmup, 3)):
        fn(i)
    torch.cuda.synchronize()
    total = 0.0
    with ClockSampler(0) as clocks:
        for i in range(args.steps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(i)
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
    ms = total / args.steps
    peak, peak_src = peaks()
    achieved = algo / (ms / 1e3) / 1e9
    print(json.dumps({
        "metric": "rows_per_s", "value": rows / (ms / 1e3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if w.startswith("c5") else "f32", "data": "synthetic",
        "config": {"workload": w, "rows": rows, "row_length": n, "l2": "256 MB flush buffer written between steps"},
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "note": note}}), flush=True)


def vocab_sharded_record(args, torch, dist, device, rank, world, steps=30):
    """Configuration 5: bf16 [1024, 151936] sharded along the vocabulary over the ranks (strong scaling).
    One step = local top-k' per shard, exchange of the candidates, merge and sample.  The exchange is timed
    both ways: done by the candidate kernel over peer memory (the record's headline) and as an NCCL all-gather
    between the two kernels.  Returns the record on rank 0, None elsewhere.  The process group (if world > 1)
    is the caller's."""
    from tallax_b200 import _lib, sampling
    lib = _lib.load()
    rows, vocab, k = 1024, 151936, 50
    vl = vocab // world
    # every rank draws the same full matrix (same seed) and keeps its slice; rank 0 keeps all of it for the check
    g = torch.Generator(device=device)
    g.manual_seed(4)
    x = torch.randn((rows, vocab), generator=g, device=device) * 2.0
    order = torch.rand((rows, vocab), generator=g, device=device).argsort(dim=1).argsort(dim=1).float() + 1.0
    x = (x + 4.0 * order.pow(-1.1)).to(torch.bfloat16)
    del order
    noise = torch.rand((rows, vocab), generator=g, device=device)
    shard = x[:, rank * vl:(rank + 1) * vl].contiguous()
    nshard = noise[:, rank * vl:(rank + 1) * vl].contiguous()
    md = sampling.SamplingMetadata(top_k=torch.full((rows,), k, dtype=torch.int32, device=device),
                                   top_p=torch.full((rows,), 0.95, device=device),
                                   temperature=torch.full((rows,), 0.8, device=device))
    vws = sampling.VocabShardedWorkspace(rows, k, world, device)
    exchange = sampling.make_vocab_exchange(rows, k, device=device)     # a collective; ends with a barrier
    mismatches = None
    if rank == 0:
        whole = sampling.sample(None, x[:, :vl * world], md, noise=noise[:, :vl * world]).clone()
    del x, noise
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)   # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_gathered():
        return sampling.sample_vocab_sharded(None, shard, md, noise_shard=nshard, k_cand=k, workspace=vws)

    def step_exchange():
        return sampling.sample_vocab_sharded(None, shard, md, noise_shard=nshard, k_cand=k, workspace=vws,
                                             exchange=exchange)

    def timed(step):
        """(ms per step as the max over ranks, clock summary, launches, tokens of the first call)"""
        tok = step().clone()
        for _ in range(max(args.warmup, 3)):
            step()
        barrier()
        total = 0.0
        launches0 = lib.tlx_kernel_launches()
        with ClockSampler(device.index) as clocks:
            for i in range(steps):
                flush.fill_(i & 0xFF)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                e1.synchronize()
                total += e0.elapsed_time(e1)
        launches = lib.tlx_kernel_launches() - launches0
        t = torch.tensor([total], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps, clocks, int(launches), tok

    # the step as a CUDA graph of the two kernels (the exchange path has no collective call to capture)
    def timed_graph():
        graph = torch.cuda.CUDAGraph()
        barrier()
        with torch.cuda.graph(graph):
            step_exchange()
        barrier()
        total = 0.0
        for i in range(steps):
            flush.fill_(i & 0xFF)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    # Steps queued back to back, as a decode loop issues them: no barrier and no host synchronisation between
    # steps, four rotating copies of the shard (rows rolled) so that every step reads from HBM once the four
    # shards exceed L2 (8 ranks: 4 x 39 MB of logits; the step's other reads are gathers).  One CUDA graph per
    # copy; the time per step is (last step's end - first step's start) / steps, max over ranks.
    def timed_back_to_back(n_steps=200):
        shards4 = [shard] + [torch.roll(shard, j, dims=0) for j in (1, 2, 3)]
        noise4 = [nshard] + [torch.roll(nshard, j, dims=0) for j in (1, 2, 3)]
        graphs = []
        for j in range(4):
            sampling.sample_vocab_sharded(None, shards4[j], md, noise_shard=noise4[j], k_cand=k, workspace=vws,
                                          exchange=exchange)
        barrier()
        for j in range(4):
            gj = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gj):
                sampling.sample_vocab_sharded(None, shards4[j], md, noise_shard=noise4[j], k_cand=k, workspace=vws,
                                              exchange=exchange)
            graphs.append(gj)
        for j in range(4):          # every rank replays the same sequence: the exchange stays in step
            graphs[j].replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            graphs[i % 4].replay()
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        barrier()
        return float(t.item()) / n_steps

    ms_g, _, launches_g, tok_g = timed(step_gathered)
    ms, clocks, launches, tok = timed(step_exchange)
    ms_graph = timed_graph()
    ms_b2b = timed_back_to_back()
    ex_steps, ex_error = exchange.state()
    barrier()
    if rank == 0:
        mismatches = int((whole != tok).sum())
        mismatches_g = int((whole != tok_g).sum())
    exchange.close()
    if rank != 0:
        return None
    peak, peak_src = peaks()
    algo = rows * vl * 2 + rows * k * 12        # this rank's logits once + its candidates out
    achieved = algo / (ms / 1e3) / 1e9
    return {
        "metric": METRIC, "value": rows / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c5: bf16 [1024,151936] = N(0,2) + 4*rank^-1.1, T=0.8, top_k=50, top_p=0.95, "
                               "vocab split over the ranks, k'=50 candidates per shard, stored by the candidate "
                               "kernel into every rank's exchange buffer over NVLink; the merge kernel waits per row",
                   "l2": "256 MB flush buffer written between steps"},
        "clocks": clocks.summary(), "gpu_launches": int(launches),
        "mismatches": mismatches,
        "parity": f"{mismatches} of {rows} tokens differ from the unsharded fused sampler on rank 0",
        "exchange_state": {"steps": ex_steps, "error": ex_error},
        "graph_replay_ms_per_step": ms_graph,
        "back_to_back": {"ms_per_step": ms_b2b, "value": rows / (ms_b2b / 1e3), "unit": UNIT, "steps": 200,
                         "note": "200 steps queued back to back as CUDA-graph replays (no barrier or host "
                                 "synchronisation between steps; four rotating copies of the shard); the figures "
                                 "above it are per-step latencies, each step started from idle after a barrier"},
        "nccl_all_gather": {"ms_per_step": ms_g, "gpu_launches": launches_g, "mismatches": mismatches_g,
                            "note": "the same step with torch.distributed all_gather_into_tensor between the two "
                                    "kernels"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src,
                     "note": "per GPU: its logits slice once + candidates, over the whole step "
                             "(candidate kernel with the exchange, merge kernel)"}}


def run_vocab_sharded(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    rec = vocab_sharded_record(args, torch, dist, device, rank, world, steps=args.steps)
    if rec is not None:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="time plain library calls instead of CUDA graph launches")
    ap.add_argument("--rows-per-call", type=int, default=0, choices=[0, 32, 64, 128],
                    help="time calls of this many rows instead of 256 (the small-batch paths)")
    ap.add_argument("--mix", default="c3", choices=["c3", "greedy", "k1", "k50", "k1024", "no-wide", "all-wide"],
                    help="c3 (default): the benchmark's parameter mix; the others keep its logits and noise and set "
                         "temperature 0 / top_k 1, 50, 1024 for every row / top_k 500 for the rows without top-k / "
                         "no top-k for any row (one GPU, kernel time only)")
    ap.add_argument("--rows", type=int, default=0, help="row count of the c5-shard-of-8 / c5-merge-of-8 workloads")
    ap.add_argument("--workload", default="c3", help="c3 (default, the fused sampler) | c1 | c2 | c4a | "
                    "c4a-single-pass | c4b: the other operators at their benchmark sizes, one GPU, rows/s | c5: the "
                    "vocab-sharded sampler over the ranks of torchrun | c5-shard-of-8, c5-merge-of-8: one rank's "
                    "two stages of an 8-way vocabulary split, on one GPU")
    args = ap.parse_args()
    if args.workload == "c5" and args.impl == "ours":
        run_vocab_sharded(args)
        return
    if args.workload != "c3" and args.impl == "ours":
        run_op_workload(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
