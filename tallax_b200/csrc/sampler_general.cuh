// Whole-row ("general") sampler paths that work on a row in global memory, whatever
// its top-k: the exact fallback of the sliced sampler and the path for rows whose top-k
// filter is disabled or larger than the single-pass limit.
//   bf16 : windowed histogram over the full 16-bit key.  The softmax mass of a value
//          group is count * exp(value - max), so counts alone give the exact top-k
//          boundary, the denominator and the top-p threshold.
//   f32  : 12/12/8-bit radix passes, counts for the top-k boundary and f64 mass bins
//          for the top-p threshold.
// Both end with a streaming Gumbel arg-max over the kept elements.
#pragma once
#include "select.cuh"

namespace tlx {

__device__ __forceinline__ void block_max_u64(uint64_t& v, SelectShared& s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    uint64_t n = shfl_xor_u64(v, o);
    v = n > v ? n : v;
  }
  __syncthreads();
  if (lane_id() == 0) reinterpret_cast<uint64_t*>(s.scan_f64)[warp_id()] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  uint64_t m = 0;
  for (int w = 0; w < nw; ++w) {
    uint64_t x = reinterpret_cast<uint64_t*>(s.scan_f64)[w];
    m = x > m ? x : m;
  }
  v = m;
  __syncthreads();
}

// (max key, lowest column holding it) of a row, as key << 32 | (0x7FFFFFFF - column).
template <int DT>
static __device__ __noinline__ uint64_t row_argmax(const typename Elem<DT>::type* __restrict__ row, int64_t n,
                                               SelectShared& s) {
  using T = typename Elem<DT>::type;
  uint64_t best = 0;
  for_each_elem<DT>(row, 0, n, [&](T v, int64_t c) {
    uint64_t x = ((uint64_t)Elem<DT>::key(v) << 32) | (uint32_t)(0x7FFFFFFF - (int32_t)c);
    best = x > best ? x : best;
  });
  block_max_u64(best, s);
  return best;
}

// ---------------------------------------------------------------------------------
// general path pieces
// ---------------------------------------------------------------------------------
// Softmax denominator over the top-k set by streaming: sum of exp(x - xmax) over keys
// > vk (all keys when !bounded); the caller adds the admitted ties.
template <int DT>
static __device__ __noinline__ double stream_mass(const typename Elem<DT>::type* __restrict__ row, int64_t n, float xmax,
                                              bool bounded, uint32_t vk, SelectShared& s) {
  using T = typename Elem<DT>::type;
  // compensated f32 sum per thread (the exp itself is f32), f64 across threads
  float sum = 0.f, comp = 0.f;
  for_each_elem<DT>(row, 0, n, [&](T v, int64_t) {
    const uint32_t key = Elem<DT>::key(v);
    if (!bounded || key > vk) {
      const float y = expf(elem_as_float<DT>(v) - xmax) - comp;
      const float t = sum + y;
      comp = (t - sum) - y;
      sum = t;
    }
  });
  const double acc = (double)sum - (double)comp;
  double total;
  block_scan_incl<double>(acc, s.scan_f64, &total, ShflUpF64());
  return total;
}

// Streaming Gumbel arg-max over the kept elements:
//   key >= vstar, and inside the top-k set: key > vk, or key == vk with tie rank < ties_admitted
// (rank = number of equal keys at lower columns).  `ordered` selects the traversal that
// tracks tie ranks; it is only needed when the kept set cuts through the tie group.
//
// The score y = x / T + gumbel(u) is screened in f32: every thread keeps its two best
// screened scores, the block maximum A is reduced, and only elements within kGumbelSlack
// of A are decided on the f64-evaluated Gumbel term.  If some thread has two elements that
// close to A (there may then be a third), the row is traversed once more instead.
template <int DT, typename F>
__device__ __forceinline__ void for_each_kept(const typename Elem<DT>::type* __restrict__ row, int64_t n,
                                              uint32_t vstar, bool bounded, uint32_t vk, uint32_t ties_admitted,
                                              bool ordered, SelectShared& s, F&& f) {
  using T = typename Elem<DT>::type;
  if (!ordered) {
    for_each_elem<DT>(row, 0, n, [&](T v, int64_t c) {
      const uint32_t key = Elem<DT>::key(v);
      if (key >= vstar && (!bounded || key >= vk)) f(elem_as_float<DT>(v), c);
    });
  } else {
    const int64_t L = (n + blockDim.x - 1) / blockDim.x;
    const int64_t b0 = (int64_t)threadIdx.x * L, b1 = (b0 + L < n) ? b0 + L : n;
    uint32_t ties = 0;
    for (int64_t c = b0; c < b1; ++c) ties += (Elem<DT>::key(row[c]) == vk);
    uint32_t tot;
    uint32_t rank = block_scan_incl<uint32_t>(ties, s.scan_u32, &tot, ShflUpU32()) - ties;
    for (int64_t c = b0; c < b1; ++c) {
      const T v = row[c];
      const uint32_t key = Elem<DT>::key(v);
      if (key > vk) { if (key >= vstar) f(elem_as_float<DT>(v), c); }
      else if (key == vk) { if (rank < ties_admitted && key >= vstar) f(elem_as_float<DT>(v), c); rank++; }
    }
  }
}

__device__ __forceinline__ Best block_best(Best best, SelectShared& s) {
  best = warp_best(best);
  __syncthreads();
  if (lane_id() == 0) { s.scan_f64[warp_id()] = (double)best.y; s.scan_u32[warp_id()] = (uint32_t)best.tok; }
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  Best b{-INFINITY, 0x7FFFFFFF};
  for (int w = 0; w < nw; ++w) b = best_of(b, Best{(float)s.scan_f64[w], (int)s.scan_u32[w]});
  __syncthreads();
  return b;
}

template <int DT>
static __device__ __noinline__ int final_argmax(const typename Elem<DT>::type* __restrict__ row, int64_t n, float T_,
                                            uint32_t vstar, bool bounded, uint32_t vk, uint32_t ties_admitted,
                                            bool ordered, const NoiseSrc& noise, int64_t nrow, SelectShared& s) {
  // screening pass: two best screened scores per thread, with what is needed to re-evaluate the best
  float a1 = -INFINITY, a2 = -INFINITY, q1 = 0.f, u1 = 0.5f;
  int c1 = 0x7FFFFFFF;
  for_each_kept<DT>(row, n, vstar, bounded, vk, ties_admitted, ordered, s, [&](float x, int64_t c) {
    const float u = noise.at(nrow, c);
    const float q = __fdiv_rn(x, T_);
    const float a = q + gumbel_screen(u);
    if (a > a1) { a2 = a1; a1 = a; q1 = q; u1 = u; c1 = (int)c; }
    else if (a > a2) a2 = a;
  });
  const Best top = block_best(Best{a1, c1}, s);
  const float cut = top.y - (kGumbelSlack + 1e-5f * fabsf(top.y));
  const int crowded = __syncthreads_or(a2 >= cut);
  Best best{-INFINITY, 0x7FFFFFFF};
  if (!crowded) {
    if (a1 >= cut) best = Best{q1 + gumbel_exact(u1), c1};
  } else {
    for_each_kept<DT>(row, n, vstar, bounded, vk, ties_admitted, ordered, s, [&](float x, int64_t c) {
      const float u = noise.at(nrow, c);
      const float q = __fdiv_rn(x, T_);
      if (q + gumbel_screen(u) >= cut) best = best_of(best, Best{q + gumbel_exact(u), (int)c});
    });
  }
  return block_best(best, s).tok;
}


// ---- bf16: 16-bit keys ---------------------------------------------------------------
__device__ __forceinline__ uint32_t key16_to_key32(uint32_t k16) {
  return (k16 << 16) | ((k16 & 0x8000u) ? 0u : 0xFFFFu);
}
__device__ __forceinline__ float key16_value(int k16) { return key_f32(key16_to_key32((uint32_t)k16)); }

// Histogram of the keys in [whi - WIN + 1, whi] into win[whi - key16].
template <int WIN>
static __device__ __noinline__ void window_hist(const __nv_bfloat16* __restrict__ row, int64_t n, int whi, uint32_t* win) {
  for (int i = threadIdx.x; i < WIN; i += blockDim.x) win[i] = 0;
  __syncthreads();
  for_each_elem<TLX_BF16>(row, 0, n, [&](__nv_bfloat16 v, int64_t) {
    const int d = whi - (int)(Elem<TLX_BF16>::key(v) >> 16);
    if (d >= 0 && d < WIN) atomicAdd(&win[d], 1u);
  });
  __syncthreads();
}

// Largest 16-bit key of the row that is <= `limit`, or -1 (also when limit < 0).  All threads call.
static __device__ __noinline__ int next_key_below(const __nv_bfloat16* __restrict__ row, int64_t n, int limit,
                                                  SelectShared& s) {
  if (limit < 0) return -1;
  uint64_t best = 0;   // key + 1, 0 = none
  for_each_elem<TLX_BF16>(row, 0, n, [&](__nv_bfloat16 v, int64_t) {
    const int k16 = (int)(Elem<TLX_BF16>::key(v) >> 16);
    if (k16 <= limit && (uint64_t)(k16 + 1) > best) best = (uint64_t)(k16 + 1);
  });
  block_max_u64(best, s);
  return (int)best - 1;
}

// What a caller may already know about the row (the sliced sampler assembles these from
// its slices); anything absent is computed from global memory.
struct RowPreset {
  uint64_t top = 0;     // row_argmax composite, 0 = unknown
  bool have_window = false;  // win[] already holds the histogram of the window anchored at the row maximum
  double mass = -1.0;   // sum of exp(x - max) over the WHOLE row, < 0 = unknown (used when top-k is disabled)
  bool threshold_only = false;  // top-k disabled: return the top-p threshold (16-bit key) instead of sampling
};

// One row, any top-k.  `win` holds WIN uint32 bins; blockDim.x must divide WIN.
template <int WIN>
static __device__ __noinline__ int general_row_bf16(const __nv_bfloat16* __restrict__ row, int64_t n, int K, float p_row,
                                                float T_, const NoiseSrc& noise, int64_t nrow, SelectShared& s,
                                                uint32_t* win, const RowPreset& pre) {
  const int kPer = WIN / (int)blockDim.x;  // window slots per thread, descending key order
  const bool bounded = (int64_t)K < n;
  const uint64_t top = pre.top ? pre.top : row_argmax<TLX_BF16>(row, n, s);
  const int kmax = (int)((uint32_t)(top >> 32) >> 16);
  const float xmax = key_f32((uint32_t)(top >> 32));
  int hist_whi = pre.have_window ? kmax : -1;  // window currently held in `win`

  // ---- phase A: the top-k boundary (key vk, admitted ties) by counts ------------------
  int vk16 = -1;
  uint32_t ties_admitted = 0, ties_total = 0;
  if (bounded) {
    uint32_t cnt_hi = 0;
    for (int whi = kmax; whi >= 0; whi -= WIN) {
      if (hist_whi != whi) { window_hist<WIN>(row, n, whi, win); hist_whi = whi; }
      uint32_t local = 0;
      const int i0 = threadIdx.x * kPer;
      for (int j = 0; j < kPer; ++j) local += win[i0 + j];
      uint32_t total;
      const uint32_t incl = block_scan_incl<uint32_t>(local, s.scan_u32, &total, ShflUpU32());
      const uint32_t before = cnt_hi + incl - local;
      if (before < (uint32_t)K && before + local >= (uint32_t)K) {
        uint32_t run = before;
        for (int j = 0; j < kPer; ++j) {
          const uint32_t c = win[i0 + j];
          if (run + c >= (uint32_t)K) {
            s.tmp_i[0] = whi - (i0 + j);
            s.tmp_i[1] = (int)((uint32_t)K - run);
            s.tmp_i[2] = (int)c;
            break;
          }
          run += c;
        }
      }
      __syncthreads();
      if (cnt_hi + total >= (uint32_t)K) {
        vk16 = s.tmp_i[0];
        ties_admitted = (uint32_t)s.tmp_i[1];
        ties_total = (uint32_t)s.tmp_i[2];
        __syncthreads();
        break;
      }
      cnt_hi += total;
      __syncthreads();
    }
  }
  const uint32_t vk32 = vk16 >= 0 ? key16_to_key32((uint32_t)vk16) : 0u;

  // ---- phase B: softmax denominator over the top-k set ---------------------------------
  double Z;
  if (!bounded && pre.mass >= 0.0) {
    Z = pre.mass;
  } else {
    Z = stream_mass<TLX_BF16>(row, n, xmax, bounded, vk32, s);
    if (bounded) Z += (double)ties_admitted * (double)expf(key_f32(vk32) - xmax);
  }
  const double target = (double)p_row * Z;

  // ---- phase C: top-p threshold = first value group (descending) whose cumulative mass
  //      over the top-k set reaches top_p * Z -----------------------------------------------
  int vstar16 = bounded ? vk16 : 0;
  {
    double cum = 0.0;
    const int lowest = bounded ? vk16 : 0;
    for (int whi = kmax; whi >= lowest;) {
      if (hist_whi != whi) { window_hist<WIN>(row, n, whi, win); hist_whi = whi; }
      const int i0 = threadIdx.x * kPer;
      double local = 0.0;
      for (int j = 0; j < kPer; ++j) {
        const int k16 = whi - (i0 + j);
        uint32_t c = win[i0 + j];
        if (bounded) { if (k16 < vk16) c = 0; else if (k16 == vk16) c = ties_admitted; }
        if (c && k16 >= 0) local += (double)c * (double)expf(key16_value(k16) - xmax);
      }
      double total;
      const double incl = block_scan_incl<double>(local, s.scan_f64, &total, ShflUpF64());
      const double before = cum + incl - local;
      if (threadIdx.x == 0) s.tmp_i[3] = -1;
      __syncthreads();
      if (before < target && before + local >= target) {
        double run = before;
        for (int j = 0; j < kPer; ++j) {
          const int k16 = whi - (i0 + j);
          uint32_t c = win[i0 + j];
          if (bounded) { if (k16 < vk16) c = 0; else if (k16 == vk16) c = ties_admitted; }
          if (c && k16 >= 0) {
            run += (double)c * (double)expf(key16_value(k16) - xmax);
            if (run >= target) { s.tmp_i[3] = k16; break; }
          }
        }
      }
      __syncthreads();
      const int found = s.tmp_i[3];
      __syncthreads();
      if (found >= 0) { vstar16 = found; break; }
      cum += total;
      // the next window hangs from the largest key present below this one (the keys in between,
      // e.g. the denormal range between the positive and the negative values, are skipped)
      whi = next_key_below(row, n, whi - WIN, s);
    }
  }
  if (pre.threshold_only && !bounded) return vstar16;
  const uint32_t vstar32 = vstar16 == 0 ? 0u : key16_to_key32((uint32_t)vstar16);
  const bool ordered = bounded && vstar16 == vk16 && ties_admitted < ties_total;
  return final_argmax<TLX_BF16>(row, n, T_, vstar32, bounded, vk32, ties_admitted, ordered, noise, nrow, s);
}

// ---- any float dtype: 32-bit keys, radix digits of 12 / 12 / 8 bits -----------------------
// `mass` holds kHistBins doubles; blockDim.x must divide kHistBins.
template <int DT>
static __device__ __noinline__ int general_row_radix(const typename Elem<DT>::type* __restrict__ row, int64_t n, int K,
                                                 float p_row, float T_, const NoiseSrc& noise, int64_t nrow,
                                                 SelectShared& s, double* mass) {
  using T = typename Elem<DT>::type;
  const int kPer = kHistBins / (int)blockDim.x;
  const int shifts[3] = {20, 8, 0};
  const int bits[3] = {12, 12, 8};
  const bool bounded = (int64_t)K < n;
  const uint64_t top = row_argmax<DT>(row, n, s);
  const float xmax = key_f32((uint32_t)(top >> 32));

  // phase A: K-th largest key and the number of admitted ties, by counting passes
  uint32_t vk = 0, ties_admitted = 0, ties_total = 0;
  if (bounded) {
    uint32_t prefix = 0, prefix_mask = 0;
    int need = K;
    for (int d = 0; d < 3; ++d) {
      const int nb = 1 << bits[d], sh = shifts[d];
      for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) s.hist[i] = 0;
      __syncthreads();
      for_each_elem<DT>(row, 0, n, [&](T v, int64_t) {
        const uint32_t key = Elem<DT>::key(v);
        if ((key & prefix_mask) == prefix) atomicAdd(&s.hist[(key >> sh) & (nb - 1)], 1u);
      });
      __syncthreads();
      find_threshold_bin(s, need, 0);
      const int b = s.bin, above = s.above;
      const uint32_t cb = s.hist[b];
      __syncthreads();
      prefix |= (uint32_t)b << sh;
      prefix_mask |= (uint32_t)(nb - 1) << sh;
      need -= above;
      ties_total = cb;
    }
    vk = prefix;
    ties_admitted = (uint32_t)need;
  }

  // phase B: softmax denominator over the top-k set
  double Z = stream_mass<DT>(row, n, xmax, bounded, vk, s);
  const double wk = bounded ? (double)expf(key_f32(vk) - xmax) : 0.0;
  if (bounded) Z += (double)ties_admitted * wk;
  const double target = (double)p_row * Z;

  // phase C: radix descent on cumulative mass
  uint32_t vstar;
  {
    uint32_t prefix = 0, prefix_mask = 0;
    double cum = 0.0;
    bool fell_through = false;
    for (int d = 0; d < 3 && !fell_through; ++d) {
      const int nb = 1 << bits[d], sh = shifts[d];
      for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) mass[i] = 0.0;
      __syncthreads();
      for_each_elem<DT>(row, 0, n, [&](T v, int64_t) {
        const uint32_t key = Elem<DT>::key(v);
        if ((key & prefix_mask) == prefix && (!bounded || key > vk))
          atomicAdd(&mass[(key >> sh) & (nb - 1)], (double)expf(elem_as_float<DT>(v) - xmax));
      });
      __syncthreads();
      if (threadIdx.x == 0 && bounded && (vk & prefix_mask) == prefix)
        mass[(vk >> sh) & (nb - 1)] += (double)ties_admitted * wk;
      if (threadIdx.x == 0) s.tmp_i[3] = -1;
      __syncthreads();
      // thread t owns bins [hi - kPer + 1, hi] in descending order
      const int hi = kHistBins - 1 - threadIdx.x * kPer;
      double local = 0.0;
      for (int j = 0; j < kPer; ++j) local += mass[hi - j];
      double total;
      const double incl = block_scan_incl<double>(local, s.scan_f64, &total, ShflUpF64());
      const double before = cum + incl - local;
      if (before < target && before + local >= target) {
        double run = before;
        for (int j = 0; j < kPer; ++j) {
          const double mj = mass[hi - j];
          if (mj > 0.0 && run + mj >= target) {
            s.tmp_i[3] = hi - j;
            s.scan_f64[36] = run;
            break;
          }
          run += mj;
        }
      }
      __syncthreads();
      const int found = s.tmp_i[3];
      const double cum_before = s.scan_f64[36];
      __syncthreads();
      if (found < 0) { fell_through = true; break; }
      prefix |= (uint32_t)found << sh;
      prefix_mask |= (uint32_t)(nb - 1) << sh;
      cum = cum_before;
    }
    // Mass short of the target (top_p ~ 1 and rounding): keep the whole top-k set.
    vstar = fell_through ? (bounded ? vk : 0u) : prefix;
  }
  const bool ordered = bounded && vstar == vk && ties_admitted < ties_total;
  return final_argmax<DT>(row, n, T_, vstar, bounded, vk, ties_admitted, ordered, noise, nrow, s);
}

}  // namespace tlx
