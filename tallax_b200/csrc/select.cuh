// Row-wise selection building blocks shared by the top-k and sampler kernels.
//
// 1. collect_row: ONE streaming pass over a row that leaves in shared memory a small
//    superset of the row's top-K.  A 4096-bin histogram of the top 12 key bits is kept
//    for the bins at or above a threshold bin B; B is the largest bin such that at
//    least K elements seen so far lie in bins >= B, so it only ever rises and an
//    element below it can never be in the top-K.  Elements at or above B are appended
//    to the candidate list, which is re-filtered whenever B rises.  Exact, not
//    probabilistic; the only failure is a candidate-list overflow (e.g. an ascending
//    row or a huge group of equal values), reported to the caller.
// 2. exact_select_row: multi-pass radix select over global memory, the fallback.
// 3. sample_tail: softmax mass, top-p threshold, temperature, Gumbel arg-max over
//    sorted candidates.
#pragma once
#include "tlx_common.cuh"

namespace tlx {

constexpr int kHistBins = 4096;   // top 12 bits of the 32-bit key
constexpr int kHistShift = 20;
constexpr int kFirstChunk = 8192; // elements histogrammed in full before filtering starts

// Candidate composite: (~key) << 32 | low, so ascending u64 order is (key desc, low asc).
__device__ __forceinline__ uint64_t cand_make(uint32_t key, uint32_t low) { return ((uint64_t)(~key) << 32) | low; }
__device__ __forceinline__ uint32_t cand_key(uint64_t c) { return ~(uint32_t)(c >> 32); }
__device__ __forceinline__ uint32_t cand_low(uint64_t c) { return (uint32_t)c; }

struct SelectShared {
  uint32_t hist[kHistBins];
  uint32_t scan_u32[40];
  double scan_f64[40];
  int fill;       // candidates appended (may exceed capacity: overflow)
  int bin;        // current threshold bin B
  int above;      // elements in bins > B at the last refinement
  int refinements;
  int tmp_i[4];
  unsigned long long tmp_u64[2];
  float tmp_f[4];
};

// Real value at the lower edge of histogram bin b, clamped so that it is never a NaN
// pattern: a float compare against it passes a superset of "bin >= b".
__device__ __forceinline__ float bin_lower_value(int b) {
  if (b <= 7) return -INFINITY;  // -inf itself lives in bin 7
  b = min(b, 4088);
  return key_f32((uint32_t)b << kHistShift);
}

// ---- vectorised row traversal ---------------------------------------------------
// Calls f(value, column) for every column in [c0, c1), 16-byte loads in the aligned
// body, kU vectors in flight per thread.
template <int DT, int kU = 4, typename F>
__device__ __forceinline__ void for_each_elem(const typename Elem<DT>::type* __restrict__ row, int64_t c0, int64_t c1,
                                              F&& f) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  if (c1 <= c0) return;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(row + c0);
  int64_t head = (int64_t)(((16 - (addr & 15)) & 15) / sizeof(T));
  if (head > c1 - c0) head = c1 - c0;
  for (int64_t c = c0 + threadIdx.x; c < c0 + head; c += blockDim.x) f(row[c], c);
  const int64_t vb = c0 + head;
  const int64_t nvec = (c1 - vb) / VEC;
  const uint4* vp = reinterpret_cast<const uint4*>(row + vb);
  int64_t i = threadIdx.x;
  for (; i + (int64_t)(kU - 1) * blockDim.x < nvec; i += (int64_t)kU * blockDim.x) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) v[u] = __ldg(vp + i + (int64_t)u * blockDim.x);
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const T* e = reinterpret_cast<const T*>(&v[u]);
      const int64_t cb = vb + (i + (int64_t)u * blockDim.x) * VEC;
#pragma unroll
      for (int j = 0; j < VEC; ++j) f(e[j], cb + j);
    }
  }
  for (; i < nvec; i += blockDim.x) {
    uint4 v = __ldg(vp + i);
    const T* e = reinterpret_cast<const T*>(&v);
    const int64_t cb = vb + i * VEC;
#pragma unroll
    for (int j = 0; j < VEC; ++j) f(e[j], cb + j);
  }
  for (int64_t c = vb + nvec * VEC + threadIdx.x; c < c1; c += blockDim.x) f(row[c], c);
}

template <int DT>
__device__ __forceinline__ float elem_as_float(typename Elem<DT>::type v) {
  if constexpr (DT == TLX_F32) return v;
  else if constexpr (DT == TLX_BF16) return __bfloat162float(v);
  else if constexpr (DT == TLX_F16) return __half2float(v);
  else return 0.f;
}

// ---- threshold refinement -------------------------------------------------------
// Largest bin B with (#elements in bins >= B) >= K, from the histogram; 0 if fewer
// than K elements were counted.  Also returns the count in bins > B.  All threads call.
static __device__ __noinline__ void find_threshold_bin(SelectShared& s, int K, int lower_bound_bin) {
  const int nt = blockDim.x;
  const int per = kHistBins / nt;  // blockDim divides 4096
  // thread t owns the bins [hi - per + 1, hi], hi = 4095 - t*per (descending order)
  const int hi = kHistBins - 1 - threadIdx.x * per;
  uint32_t local = 0;
  for (int j = 0; j < per; ++j) local += s.hist[hi - j];
  uint32_t total;
  uint32_t incl = block_scan_incl<uint32_t>(local, s.scan_u32, &total, ShflUpU32());
  const uint32_t excl = incl - local;
  if (threadIdx.x == 0 && total < (uint32_t)K) { s.bin = lower_bound_bin; s.above = 0; }
  if (excl < (uint32_t)K && incl >= (uint32_t)K) {
    uint32_t run = excl;
    for (int j = 0; j < per; ++j) {
      const uint32_t c = s.hist[hi - j];
      if (run + c >= (uint32_t)K) {
        s.bin = max(hi - j, lower_bound_bin);
        s.above = (int)run;
        break;
      }
      run += c;
    }
  }
  __syncthreads();
}

// Drop candidates whose bin fell below s.bin.  In place: every thread first reads its
// contiguous share, then (after the scan's barriers) writes the survivors.
template <int CAP>
static __device__ __noinline__ void compact_candidates(SelectShared& s, uint64_t* cand) {
  constexpr int kMaxPer = 16;
  const int n = min(s.fill, CAP);
  const int per = (n + blockDim.x - 1) / blockDim.x;  // <= CAP / blockDim <= kMaxPer
  const int b0 = threadIdx.x * per;
  const uint32_t min_key = (uint32_t)s.bin << kHistShift;
  uint64_t item[kMaxPer];
  uint32_t kept_mask = 0;
#pragma unroll
  for (int j = 0; j < kMaxPer; ++j) {
    item[j] = 0;
    if (j < per && b0 + j < n) {
      item[j] = cand[b0 + j];
      if (cand_key(item[j]) >= min_key) kept_mask |= 1u << j;
    }
  }
  const int nk = __popc(kept_mask);
  uint32_t total;
  uint32_t incl = block_scan_incl<uint32_t>((uint32_t)nk, s.scan_u32, &total, ShflUpU32());
  int o = (int)(incl - nk);
#pragma unroll
  for (int j = 0; j < kMaxPer; ++j)
    if (kept_mask & (1u << j)) cand[o++] = item[j];
  if (threadIdx.x == 0) s.fill = (int)total;
  __syncthreads();
}

// ---- the streaming collector ----------------------------------------------------
// After the call: cand[0 .. s.fill) holds every element of the row whose bin >= s.bin,
// which includes the whole top-K (K <= CAP/4 expected).  Returns false on overflow (the
// list then holds an arbitrary subset).  `low_of(column)` is stored in the composite's
// low word.  Requires blockDim.x to divide 4096 and CAP <= 16 * blockDim.x.
template <int DT, int CAP>
__device__ __forceinline__ bool collect_row(const typename Elem<DT>::type* __restrict__ row, int64_t n, int K,
                                            SelectShared& s, uint64_t* cand) {
  using T = typename Elem<DT>::type;
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) s.hist[i] = 0;
  if (threadIdx.x == 0) { s.fill = 0; s.bin = 0; s.above = 0; s.refinements = 0; }
  __syncthreads();
  const int64_t n0 = n < kFirstChunk ? n : (int64_t)kFirstChunk;
  for_each_elem<DT>(row, 0, n0, [&](T v, int64_t) { atomicAdd(&s.hist[Elem<DT>::key(v) >> kHistShift], 1u); });
  __syncthreads();
  find_threshold_bin(s, K, 0);

  auto push = [&](uint32_t key, int64_t c) {
    const int slot = atomicAdd(&s.fill, 1);
    if (slot < CAP) cand[slot] = cand_make(key, (uint32_t)c);
  };
  auto refine = [&]() {
    __syncthreads();
    const int old_bin = s.bin;
    __syncthreads();
    find_threshold_bin(s, K, old_bin);
    if (s.bin != old_bin) {
      if (threadIdx.x == 0) s.refinements++;
      compact_candidates<CAP>(s, cand);
    }
  };

  // the first chunk again, now filtered (its elements are already in the histogram)
  {
    const int bin = s.bin;
    if constexpr (DT == TLX_I32 || DT == TLX_U32) {
      for_each_elem<DT>(row, 0, n0, [&](T v, int64_t c) {
        const uint32_t key = Elem<DT>::key(v);
        if ((int)(key >> kHistShift) >= bin) push(key, c);
      });
    } else {
      const float thr = bin_lower_value(bin);
      for_each_elem<DT>(row, 0, n0, [&](T v, int64_t c) {
        if (!(elem_as_float<DT>(v) < thr)) {
          const uint32_t key = Elem<DT>::key(v);
          if ((int)(key >> kHistShift) >= bin) push(key, c);
        }
      });
    }
  }
  // the rest of the row in intervals that double in length, refining B in between
  int64_t done = n0;
  while (done < n) {
    int64_t upto = done * 2;
    if (upto > n) upto = n;
    __syncthreads();
    const int bin = s.bin;
    if constexpr (DT == TLX_I32 || DT == TLX_U32) {
      for_each_elem<DT, 8>(row, done, upto, [&](T v, int64_t c) {
        const uint32_t key = Elem<DT>::key(v);
        if ((int)(key >> kHistShift) >= bin) {
          atomicAdd(&s.hist[key >> kHistShift], 1u);
          push(key, c);
        }
      });
    } else {
      const float thr = bin_lower_value(bin);
      for_each_elem<DT, 8>(row, done, upto, [&](T v, int64_t c) {
        if (!(elem_as_float<DT>(v) < thr)) {
          const uint32_t key = Elem<DT>::key(v);
          if ((int)(key >> kHistShift) >= bin) {
            atomicAdd(&s.hist[key >> kHistShift], 1u);
            push(key, c);
          }
        }
      });
    }
    done = upto;
    __syncthreads();
    if (s.fill > CAP) return false;
    refine();
  }
  __syncthreads();
  return s.fill <= CAP;
}

// ---- exact fallback: radix select over global memory ------------------------------
// Finds the K-th largest key of the row (K <= n), the number of strictly greater
// elements, and fills cand[] with exactly the top-K: all greater elements plus the
// lowest-indexed ties.  Digits of 12, 12 and 8 bits; 3 counting passes + 2 passes for
// the ordered collection.  Slow, but independent of the data's order or tie structure.
template <int DT>
static __device__ __noinline__ void exact_select_row(const typename Elem<DT>::type* __restrict__ row, int64_t n, int K,
                                                 SelectShared& s, uint64_t* cand) {
  using T = typename Elem<DT>::type;
  uint32_t prefix = 0, prefix_mask = 0;
  int need = K;  // rank still to find inside the current prefix
  const int shifts[3] = {20, 8, 0};
  const int bits[3] = {12, 12, 8};
  for (int d = 0; d < 3; ++d) {
    const int nb = 1 << bits[d];
    for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) s.hist[i] = 0;
    __syncthreads();
    const int sh = shifts[d];
    for_each_elem<DT>(row, 0, n, [&](T v, int64_t) {
      const uint32_t key = Elem<DT>::key(v);
      if ((key & prefix_mask) == prefix) atomicAdd(&s.hist[(key >> sh) & (nb - 1)], 1u);
    });
    __syncthreads();
    // bins above nb are zero, so the 4096-bin scan works for the 8-bit digit as well
    find_threshold_bin(s, need, 0);
    const int b = s.bin, above = s.above;
    __syncthreads();
    prefix |= (uint32_t)b << sh;
    prefix_mask |= (uint32_t)(nb - 1) << sh;
    need -= above;
  }
  const uint32_t vk = prefix;  // the K-th largest key; `need` ties are admitted, lowest index first
  // ordered collection: thread t owns the contiguous segment [t*L, (t+1)*L)
  const int64_t L = (n + blockDim.x - 1) / blockDim.x;
  const int64_t b0 = (int64_t)threadIdx.x * L, b1 = (b0 + L < n) ? b0 + L : n;
  uint32_t ties = 0, greater = 0;
  for (int64_t c = b0; c < b1; ++c) {
    const uint32_t key = Elem<DT>::key(row[c]);
    ties += (key == vk);
    greater += (key > vk);
  }
  uint32_t tot_t, tot_g;
  uint32_t tie_base = block_scan_incl<uint32_t>(ties, s.scan_u32, &tot_t, ShflUpU32()) - ties;
  uint32_t gt_base = block_scan_incl<uint32_t>(greater, s.scan_u32, &tot_g, ShflUpU32()) - greater;
  // layout: [greater elements in index order][admitted ties in index order]
  for (int64_t c = b0; c < b1; ++c) {
    const uint32_t key = Elem<DT>::key(row[c]);
    if (key > vk) cand[gt_base++] = cand_make(key, (uint32_t)c);
    else if (key == vk) {
      if (tie_base < (uint32_t)need) cand[tot_g + tie_base] = cand_make(key, (uint32_t)c);
      tie_base++;
    }
  }
  if (threadIdx.x == 0) { s.fill = K; s.bin = (int)(vk >> kHistShift); }
  __syncthreads();
}

// Pads cand[m .. P) with the greatest composite and sorts; returns P (power of two >= m).
static __device__ __noinline__ int sort_candidates(uint64_t* cand, int m) {
  int P = 2;
  while (P < m) P <<= 1;
  for (int i = m + threadIdx.x; i < P; i += blockDim.x) cand[i] = ~0ull;
  __syncthreads();
  block_bitonic_sort_u64(cand, P);
  return P;
}

// ---- sampler tail -----------------------------------------------------------------
// Candidates i in [0, K) are the row's top-k set in (value desc, token asc) order;
// value_of(i), token_of(i), noise_of(i) read them.  Computes
//   e_i = exp(x_i - x_0), cs = cumsum(e) / sum(e), t = min(#(cs < p), K-1),
//   keep x_i >= x_t, y_i = x_i / T + gumbel(u_i), token = arg-max y (ties: lower token).
// The arg-max is screened in f32 and decided on the f64-evaluated Gumbel term for the
// contenders only.  All threads call; the result is valid in every thread.
//
// sample_tail<kMaxItems> keeps a thread's candidates in registers and serves K <= kMaxItems *
// blockDim.x; above that it hands over to sample_tail_any, which serves any K by reading the
// candidates again in every pass (the same sums in the same order, so both give the same token).
template <typename ValueOf, typename TokenOf, typename NoiseOf>
static __device__ __noinline__ int sample_tail_any(int K, float p, float T, SelectShared& s, ValueOf value_of,
                                               TokenOf token_of, NoiseOf noise_of) {
  const int per = (K + blockDim.x - 1) / blockDim.x;
  const int i0 = threadIdx.x * per;
  const int i1 = min(i0 + per, K);
  const int nw = (blockDim.x + 31) >> 5;
  const float x0 = value_of(0);
  double acc = 0.0;
  for (int i = i0; i < i1; ++i) acc += (double)expf(value_of(i) - x0);
  double Z;
  const double base = block_scan_incl<double>(acc, s.scan_f64, &Z, ShflUpF64()) - acc;
  int below = 0;
  const double pd = (double)p;
  double run = 0.0;
  for (int i = i0; i < i1; ++i) {
    run += (double)expf(value_of(i) - x0);
    below += ((base + run) / Z < pd) ? 1 : 0;
  }
  uint32_t t_total;
  block_scan_incl<uint32_t>((uint32_t)below, s.scan_u32, &t_total, ShflUpU32());
  const int t = min((int)t_total, K - 1);
  const float thr = value_of(t);
  float amax = -INFINITY;
  for (int i = i0; i < i1; ++i) {
    const float x = value_of(i);
    if (x >= thr) amax = fmaxf(amax, __fdiv_rn(x, T) + gumbel_screen(noise_of(i)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  __syncthreads();
  if (lane_id() == 0) s.scan_f64[warp_id()] = (double)amax;
  __syncthreads();
  amax = -INFINITY;
  for (int w = 0; w < nw; ++w) amax = fmaxf(amax, (float)s.scan_f64[w]);
  __syncthreads();
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  Best best{-INFINITY, 0x7FFFFFFF};
  for (int i = i0; i < i1; ++i) {
    const float x = value_of(i);
    if (x >= thr) {
      const float u = noise_of(i);
      if (__fdiv_rn(x, T) + gumbel_screen(u) >= cut) best = best_of(best, Best{__fdiv_rn(x, T) + gumbel_exact(u), token_of(i)});
    }
  }
  best = warp_best(best);
  if (lane_id() == 0) { s.scan_f64[warp_id()] = (double)best.y; s.scan_u32[warp_id()] = (uint32_t)best.tok; }
  __syncthreads();
  Best b{-INFINITY, 0x7FFFFFFF};
  for (int w = 0; w < nw; ++w) b = best_of(b, Best{(float)s.scan_f64[w], (int)s.scan_u32[w]});
  __syncthreads();
  return b.tok;
}

template <int kMaxItems, typename ValueOf, typename TokenOf, typename NoiseOf>
static __device__ __noinline__ int sample_tail(int K, float p, float T, SelectShared& s, ValueOf value_of,
                                           TokenOf token_of, NoiseOf noise_of) {
  const int per = (K + blockDim.x - 1) / blockDim.x;
  if (per > kMaxItems) return sample_tail_any(K, p, T, s, value_of, token_of, noise_of);
  const int i0 = threadIdx.x * per;
  const float x0 = value_of(0);
  float x[kMaxItems];
  double run[kMaxItems];
  double acc = 0.0;
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < K) {
      x[j] = value_of(i);
      acc += (double)expf(x[j] - x0);
      run[j] = acc;
    }
  }
  double Z;
  const double base = block_scan_incl<double>(acc, s.scan_f64, &Z, ShflUpF64()) - acc;
  int below = 0;
  const double pd = (double)p;
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < K) below += ((base + run[j]) / Z < pd) ? 1 : 0;
  }
  uint32_t t_total;
  block_scan_incl<uint32_t>((uint32_t)below, s.scan_u32, &t_total, ShflUpU32());
  const int t = min((int)t_total, K - 1);
  const float thr = value_of(t);
  // screening pass
  float u[kMaxItems];
  float a[kMaxItems];
  float amax = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    a[j] = -INFINITY;
    if (j < per && i < K && x[j] >= thr) {
      u[j] = noise_of(i);
      a[j] = __fdiv_rn(x[j], T) + gumbel_screen(u[j]);
      amax = fmaxf(amax, a[j]);
    }
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 16));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 8));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  if (lane_id() == 0) s.scan_f64[warp_id()] = (double)amax;
  __syncthreads();
  {
    const int nw = (blockDim.x + 31) >> 5;
    float m = -INFINITY;
    for (int w = 0; w < nw; ++w) m = fmaxf(m, (float)s.scan_f64[w]);
    amax = m;
  }
  __syncthreads();
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  Best best{-INFINITY, 0x7FFFFFFF};
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < K && a[j] >= cut) {
      Best c{__fdiv_rn(x[j], T) + gumbel_exact(u[j]), token_of(i)};
      best = best_of(best, c);
    }
  }
  best = warp_best(best);
  if (lane_id() == 0) { s.scan_f64[warp_id()] = (double)best.y; s.scan_u32[warp_id()] = (uint32_t)best.tok; }
  __syncthreads();
  {
    const int nw = (blockDim.x + 31) >> 5;
    Best b{-INFINITY, 0x7FFFFFFF};
    for (int w = 0; w < nw; ++w) b = best_of(b, Best{(float)s.scan_f64[w], (int)s.scan_u32[w]});
    best = b;
  }
  __syncthreads();
  return best.tok;
}

}  // namespace tlx
