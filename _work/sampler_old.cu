// Fused temperature / top-k / top-p / noise sampler on [rows, vocab] logits, the
// candidate-level sampler, and the merge stage of the vocab-sharded sampler.
//
// tlx_sample runs two kernels on the caller's stream:
//   fast kernel    : one CTA per row.  Greedy rows need only an arg-max.  Rows with
//                    1 <= top_k <= kFastK stream the row ONCE (collect_row), sort the few
//                    candidates in shared memory and finish there (sample_tail).  Every
//                    other row (top-k disabled or large, or a candidate overflow) is
//                    appended to a work list in the workspace.
//   general kernel : persistent CTAs drain the work list.  bf16 rows use a windowed
//                    histogram over the full 16-bit key (softmax mass of a value group is
//                    count * exp(value - max), so counts alone give the exact top-p
//                    threshold); f32 rows use 12/12/8-bit radix passes with f64 mass bins.
//                    Both end with a streaming Gumbel arg-max over the kept elements.
#include <mutex>

#include "select.cuh"

namespace tlx {

constexpr int kFastThreads = 512;
constexpr int kFastCap = 4096;
constexpr int kFastK = 1024;       // largest top_k served by the single-pass kernel
constexpr int kGenThreads = 1024;
constexpr int kWindow = 32768;     // bf16 general path: full-key histogram window

struct SampleParams {
  const void* logits;
  int64_t rows, vocab, row_stride;
  const int32_t* top_k;
  const float* top_p;
  const float* temperature;
  NoiseSrc noise;
  int64_t dim0_offset;
  int32_t* out_tokens;
  int32_t* out_status;
  int32_t* worklist;  // [0] = count, [1 ..] = row ids
};

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
__device__ __forceinline__ uint64_t row_argmax(const typename Elem<DT>::type* __restrict__ row, int64_t n,
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

__device__ __forceinline__ void worklist_push(int32_t* wl, int32_t row) {
  const int slot = atomicAdd(wl, 1);
  wl[1 + slot] = row;
}

// ---------------------------------------------------------------------------------
// fast kernel
// ---------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kFastThreads) sample_fast_kernel(SampleParams p) {
  using T = typename Elem<DT>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  const int64_t r = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(p.logits) + r * p.row_stride;
  int K = p.top_k[r];
  if (K <= 0 || (int64_t)K >= p.vocab) K = (int)p.vocab;
  const float T_ = p.temperature[r];
  const float pp = p.top_p[r];

  if (T_ < kSamplingEps) {
    const uint64_t best = row_argmax<DT>(row, p.vocab, s);
    if (threadIdx.x == 0) {
      p.out_tokens[r] = 0x7FFFFFFF - (int32_t)(uint32_t)best;
      if (p.out_status) p.out_status[r] = 0;
    }
    return;
  }
  if (K > kFastK) {
    if (threadIdx.x == 0) worklist_push(p.worklist, (int32_t)r);
    return;
  }
  if (!collect_row<DT, kFastCap>(row, p.vocab, K, s, cand)) {
    if (threadIdx.x == 0) worklist_push(p.worklist, (int32_t)r);
    return;
  }
  const int m = s.fill;
  sort_candidates(cand, m);
  const int64_t nrow = r + p.dim0_offset;
  const int tok = sample_tail<2>(
      K, pp, T_, s, [&](int i) { return key_f32(cand_key(cand[i])); },
      [&](int i) { return (int)cand_low(cand[i]); },
      [&](int i) { return p.noise.at(nrow, (int64_t)cand_low(cand[i])); });
  if (threadIdx.x == 0) {
    p.out_tokens[r] = tok;
    if (p.out_status) p.out_status[r] = 0;
  }
}

// ---------------------------------------------------------------------------------
// general path pieces
// ---------------------------------------------------------------------------------
// Softmax denominator over the top-k set by streaming: sum of exp(x - xmax) over keys
// > vk (all keys when !bounded); the caller adds the admitted ties.
template <int DT>
__device__ __forceinline__ double stream_mass(const typename Elem<DT>::type* __restrict__ row, int64_t n, float xmax,
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
__device__ __forceinline__ int final_argmax(const typename Elem<DT>::type* __restrict__ row, int64_t n, float T_,
                                            uint32_t vstar, bool bounded, uint32_t vk, uint32_t ties_admitted,
                                            bool ordered, const NoiseSrc& noise, int64_t nrow, SelectShared& s) {
  // screening pass: two best screened scores per thread, with what is needed to re-evaluate the best
  float a1 = -INFINITY, a2 = -INFINITY, q1 = 0.f, u1 = 0.5f;
  int c1 = 0x7FFFFFFF;
  for_each_kept<DT>(row, n, vstar, bounded, vk, ties_admitted, ordered, s, [&](float x, int64_t c) {
    const float u = noise.at(nrow, c);
    const float q = __fdiv_rn(x, T_);
    const float a = q + gumbel_fast(u);
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
      if (q + gumbel_fast(u) >= cut) best = best_of(best, Best{q + gumbel_exact(u), (int)c});
    });
  }
  return block_best(best, s).tok;
}

// ---- bf16: 16-bit keys ---------------------------------------------------------------
__device__ __forceinline__ uint32_t key16_to_key32(uint32_t k16) {
  return (k16 << 16) | ((k16 & 0x8000u) ? 0u : 0xFFFFu);
}

// Histogram of the keys in [whi - kWindow + 1, whi] into win[whi - key16].
__device__ __forceinline__ void window_hist(const __nv_bfloat16* __restrict__ row, int64_t n, int whi, uint32_t* win) {
  for (int i = threadIdx.x; i < kWindow; i += blockDim.x) win[i] = 0;
  __syncthreads();
  for_each_elem<TLX_BF16>(row, 0, n, [&](__nv_bfloat16 v, int64_t) {
    const int d = whi - (int)(Elem<TLX_BF16>::key(v) >> 16);
    if (d >= 0 && d < kWindow) atomicAdd(&win[d], 1u);
  });
  __syncthreads();
}

__global__ void __launch_bounds__(kGenThreads) sample_general_bf16_kernel(SampleParams p) {
  using T = __nv_bfloat16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint32_t* win = reinterpret_cast<uint32_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  constexpr int kPer = kWindow / kGenThreads;  // window slots per thread, descending key order
  const int count = p.worklist[0];
  for (int w = blockIdx.x; w < count; w += gridDim.x) {
    const int64_t r = p.worklist[1 + w];
    const T* row = reinterpret_cast<const T*>(p.logits) + r * p.row_stride;
    const int64_t n = p.vocab;
    int K = p.top_k[r];
    if (K <= 0 || (int64_t)K >= n) K = (int)n;
    const bool bounded = (int64_t)K < n;
    const float T_ = p.temperature[r];
    const double target_frac = (double)p.top_p[r];

    const uint64_t top = row_argmax<TLX_BF16>(row, n, s);
    const int kmax = (int)((uint32_t)(top >> 32) >> 16);
    const float xmax = key_f32((uint32_t)(top >> 32));

    // ---- phase A: the top-k boundary (key vk, admitted ties) by counts ----------------
    int vk16 = -1;
    uint32_t ties_admitted = 0, ties_total = 0;
    int hist_whi = -1;  // window currently held in `win`
    if (bounded) {
      uint32_t cnt_hi = 0;
      for (int whi = kmax; whi >= 0; whi -= kWindow) {
        window_hist(row, n, whi, win);
        hist_whi = whi;
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

    // ---- phase B: softmax denominator over the top-k set -------------------------------
    double Z = stream_mass<TLX_BF16>(row, n, xmax, bounded, vk32, s);
    if (bounded) Z += (double)ties_admitted * (double)expf(key_f32(vk32) - xmax);
    const double target = target_frac * Z;

    // ---- phase C: top-p threshold = first value group (descending) whose cumulative mass
    //      over the top-k set reaches top_p * Z ---------------------------------------------
    int vstar16 = bounded ? vk16 : 0;
    {
      double cum = 0.0;
      const int lowest = bounded ? vk16 : 0;
      for (int whi = kmax; whi >= lowest; whi -= kWindow) {
        if (hist_whi != whi) { window_hist(row, n, whi, win); hist_whi = whi; }
        const int i0 = threadIdx.x * kPer;
        double local = 0.0;
        for (int j = 0; j < kPer; ++j) {
          const int k16 = whi - (i0 + j);
          uint32_t c = win[i0 + j];
          if (bounded) { if (k16 < vk16) c = 0; else if (k16 == vk16) c = ties_admitted; }
          if (c && k16 >= 0) local += (double)c * (double)expf(key_f32(key16_to_key32((uint32_t)k16)) - xmax);
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
              run += (double)c * (double)expf(key_f32(key16_to_key32((uint32_t)k16)) - xmax);
              if (run >= target) { s.tmp_i[3] = k16; break; }
            }
          }
        }
        __syncthreads();
        const int found = s.tmp_i[3];
        __syncthreads();
        if (found >= 0) { vstar16 = found; break; }
        cum += total;
      }
    }
    const uint32_t vstar32 = key16_to_key32((uint32_t)vstar16) & (vstar16 == 0 ? 0u : 0xFFFFFFFFu);
    const bool ordered = bounded && vstar16 == vk16 && ties_admitted < ties_total;
    const int tok = final_argmax<TLX_BF16>(row, n, T_, vstar32, bounded, vk32, ties_admitted, ordered, p.noise,
                                           r + p.dim0_offset, s);
    if (threadIdx.x == 0) {
      p.out_tokens[r] = tok;
      if (p.out_status) p.out_status[r] = 1;
    }
    __syncthreads();
  }
}

// ---- any float dtype: 32-bit keys, radix digits of 12 / 12 / 8 bits -----------------------
template <int DT>
__global__ void __launch_bounds__(kGenThreads) sample_general_radix_kernel(SampleParams p) {
  using T = typename Elem<DT>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  double* mass = reinterpret_cast<double*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  constexpr int kPer = kHistBins / kGenThreads;
  const int shifts[3] = {20, 8, 0};
  const int bits[3] = {12, 12, 8};
  const int count = p.worklist[0];
  for (int w = blockIdx.x; w < count; w += gridDim.x) {
    const int64_t r = p.worklist[1 + w];
    const T* row = reinterpret_cast<const T*>(p.logits) + r * p.row_stride;
    const int64_t n = p.vocab;
    int K = p.top_k[r];
    if (K <= 0 || (int64_t)K >= n) K = (int)n;
    const bool bounded = (int64_t)K < n;
    const float T_ = p.temperature[r];

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
    const double target = (double)p.top_p[r] * Z;

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
    const int tok = final_argmax<DT>(row, n, T_, vstar, bounded, vk, ties_admitted, ordered, p.noise,
                                     r + p.dim0_offset, s);
    if (threadIdx.x == 0) {
      p.out_tokens[r] = tok;
      if (p.out_status) p.out_status[r] = 1;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------
// candidate-level sampler: inputs already sorted descending
// ---------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) top_p_and_sample_kernel(const typename Elem<DT>::type* __restrict__ logits,
                                                               const int32_t* __restrict__ idx, int k,
                                                               const float* __restrict__ top_p,
                                                               const float* __restrict__ temperature, NoiseSrc noise,
                                                               typename Elem<DT>::type replace, int64_t dim0_offset,
                                                               int32_t* __restrict__ out) {
  using T = typename Elem<DT>::type;
  __shared__ SelectShared s;
  const int64_t r = blockIdx.x;
  const T* x = logits + r * k;
  const int32_t* id = idx + r * k;
  const float T_ = temperature[r];
  if (T_ < kSamplingEps) {
    if (threadIdx.x == 0) out[r] = id[0];
    return;
  }
  // the top-k set is the prefix of entries that were not overwritten with the replace value
  uint32_t valid = 0;
  const float rep = elem_as_float<DT>(replace);
  for (int i = threadIdx.x; i < k; i += blockDim.x) valid += (elem_as_float<DT>(x[i]) != rep) ? 1u : 0u;
  uint32_t nv;
  block_scan_incl<uint32_t>(valid, s.scan_u32, &nv, ShflUpU32());
  const int K = nv ? (int)nv : 1;
  const int64_t nrow = r + dim0_offset;
  const int tok = sample_tail<4>(
      K, top_p[r], T_, s, [&](int i) { return elem_as_float<DT>(x[i]); }, [&](int i) { return (int)id[i]; },
      [&](int i) { return noise.at(nrow, (int64_t)id[i]); });
  if (threadIdx.x == 0) out[r] = tok;
}

// ---------------------------------------------------------------------------------
// merge stage of the vocab-sharded sampler
// ---------------------------------------------------------------------------------
constexpr int kMergeThreads = 512;
constexpr int kMergeMaxCand = 8192;

__global__ void __launch_bounds__(kMergeThreads) merge_and_sample_kernel(
    const float* __restrict__ cand_vals, const int32_t* __restrict__ cand_idx, const float* __restrict__ cand_noise,
    int n_cand, int k_per_block, int64_t block_stride, int64_t row_stride, const int32_t* __restrict__ top_k,
    const float* __restrict__ top_p, const float* __restrict__ temperature, int32_t* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  const int64_t r = blockIdx.x;
  const float* v = cand_vals + r * row_stride;
  const int32_t* id = cand_idx + r * row_stride;
  const float* un = cand_noise + r * row_stride;
  auto at = [&](uint32_t i) { return (int64_t)(i / k_per_block) * block_stride + (int64_t)(i % k_per_block); };
  // low word = position in the gathered list: shards are laid side by side in ascending
  // token order, so position order equals token order among equal values
  for (int i = threadIdx.x; i < n_cand; i += blockDim.x) cand[i] = cand_make(f32_key(v[at(i)]), (uint32_t)i);
  __syncthreads();
  sort_candidates(cand, n_cand);
  int K = top_k[r];
  if (K <= 0 || K > n_cand) K = n_cand;
  const float T_ = temperature[r];
  if (T_ < kSamplingEps) {
    if (threadIdx.x == 0) out[r] = id[at(cand_low(cand[0]))];
    return;
  }
  const int tok = sample_tail<2>(
      K, top_p[r], T_, s, [&](int i) { return key_f32(cand_key(cand[i])); },
      [&](int i) { return (int)id[at(cand_low(cand[i]))]; }, [&](int i) { return un[at(cand_low(cand[i]))]; });
  if (threadIdx.x == 0) out[r] = tok;
}

// ---------------------------------------------------------------------------------
// top-p mask on the reference's (k, B) layout: column b holds row b's candidates,
// sorted descending along axis 0.  Literal semantics, including the quirk that a
// threshold index equal to k reads as 0.0.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) top_p_mask_kernel(const float* __restrict__ x, const float* __restrict__ p,
                                                         int k, int64_t B, float replace, float* __restrict__ out) {
  __shared__ double scan_f64[40];
  __shared__ uint32_t scan_u32[40];
  constexpr int kMaxItems = 8;
  const int64_t b = blockIdx.x;
  const int per = (k + blockDim.x - 1) / blockDim.x;
  const int i0 = threadIdx.x * per;
  const float x0 = x[b];
  double run[kMaxItems];
  float xv[kMaxItems];
  double acc = 0.0;
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < k) {
      xv[j] = x[(int64_t)i * B + b];
      acc += (double)expf(xv[j] - x0);
      run[j] = acc;
    }
  }
  double Z;
  const double base = block_scan_incl<double>(acc, scan_f64, &Z, ShflUpF64()) - acc;
  uint32_t below = 0;
  const double pd = (double)p[b];
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < k) below += ((base + run[j]) / Z < pd) ? 1u : 0u;
  }
  uint32_t t;
  block_scan_incl<uint32_t>(below, scan_u32, &t, ShflUpU32());
  const float thr = ((int)t < k) ? x[(int64_t)t * B + b] : 0.0f;
#pragma unroll
  for (int j = 0; j < kMaxItems; ++j) {
    const int i = i0 + j;
    if (j < per && i < k) out[(int64_t)i * B + b] = (xv[j] >= thr) ? xv[j] : replace;
  }
}

// ---------------------------------------------------------------------------------
// Gumbel arg-max with noise indexed by (idx0, idx1): position of the winner along `axis`
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gumbel_argmax_kernel(const float* __restrict__ logits,
                                                            const int32_t* __restrict__ idx0,
                                                            const int32_t* __restrict__ idx1, int64_t rows,
                                                            int64_t cols, uint32_t k0, uint32_t k1, int64_t dim1,
                                                            int axis, int32_t* __restrict__ out) {
  __shared__ float sy[8];
  __shared__ int sp[8];
  const int64_t line = blockIdx.x;                    // row (axis 1) or column (axis 0)
  const int64_t len = axis == 1 ? cols : rows;
  const int64_t step = axis == 1 ? 1 : cols;
  const int64_t start = axis == 1 ? line * cols : line;
  Best best{-INFINITY, 0x7FFFFFFF};
  for (int64_t i = threadIdx.x; i < len; i += blockDim.x) {
    const int64_t e = start + i * step;
    const float f = threefry_uniform01(k0, k1, (uint32_t)((int64_t)idx0[e] * dim1 + (int64_t)idx1[e]));
    const float u = fmaxf(f, kF32Tiny);
    const float l = logits[e];
    const float a = l + gumbel_fast(u);
    if (a >= best.y - (kGumbelSlack + 1e-5f * fabsf(best.y)) || best.y == -INFINITY)
      best = best_of(best, Best{l + gumbel_exact(u), (int)i});
  }
  best = warp_best(best);
  if (lane_id() == 0) { sy[warp_id()] = best.y; sp[warp_id()] = best.tok; }
  __syncthreads();
  if (threadIdx.x == 0) {
    Best b{-INFINITY, 0x7FFFFFFF};
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) b = best_of(b, Best{sy[w], sp[w]});
    out[line] = b.tok;
  }
}

// Raises a kernel's dynamic shared memory limit once per (kernel, device).
static int ensure_smem(const void* func, size_t bytes, const char* what) {
  struct Entry { const void* func; int dev; size_t bytes; };
  static Entry cache[256];
  static int used = 0;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].func == func && cache[i].dev == dev && cache[i].bytes >= bytes) return TLX_OK;
  cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "%s: cudaFuncSetAttribute(%zu): %s", what, bytes, cudaGetErrorString(e));
  if (used < 256) cache[used++] = Entry{func, dev, bytes};
  return TLX_OK;
}

constexpr size_t kSharedHeader = (sizeof(SelectShared) + 15) & ~size_t(15);

}  // namespace tlx

using namespace tlx;

extern "C" {

size_t tlx_sample_workspace_bytes(int64_t rows, int64_t) { return rows > 0 ? (size_t)(rows + 1) * sizeof(int32_t) : 0; }

int tlx_sample(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab, int64_t row_stride,
               const int32_t* top_k, const float* top_p, const float* temperature, const float* noise,
               int64_t noise_stride, uint32_t key0, uint32_t key1, int64_t dim0_offset, int32_t* out_tokens,
               int32_t* out_status, void* workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && vocab >= 1, "sample: bad extent");
  TLX_CHECK_ARG(vocab < (1ll << 31) && rows < (1ll << 31), "sample: extent too large");
  TLX_CHECK_ARG(row_stride >= vocab, "sample: row stride smaller than the row");
  if (dtype != TLX_F32 && dtype != TLX_BF16)
    return set_error(TLX_ERR_UNSUPPORTED, "sample: logits dtype %d not supported (f32, bf16)", dtype);
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(logits && top_k && top_p && temperature && out_tokens, "sample: null pointer");
  TLX_CHECK_ARG(!noise || noise_stride >= vocab, "sample: noise stride smaller than the row");
  const size_t need = tlx_sample_workspace_bytes(rows, vocab);
  if (!workspace || workspace_bytes < need)
    return set_error(TLX_ERR_WORKSPACE, "sample: workspace of %zu bytes needed, %zu given", need, workspace_bytes);

  SampleParams p{};
  p.logits = logits; p.rows = rows; p.vocab = vocab; p.row_stride = row_stride;
  p.top_k = top_k; p.top_p = top_p; p.temperature = temperature;
  p.noise.dense = noise; p.noise.stride = noise_stride; p.noise.k0 = key0; p.noise.k1 = key1; p.noise.vocab = vocab;
  p.dim0_offset = dim0_offset; p.out_tokens = out_tokens; p.out_status = out_status;
  p.worklist = (int32_t*)workspace;

  cudaError_t e = cudaMemsetAsync(workspace, 0, sizeof(int32_t), st);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "sample: cudaMemsetAsync: %s", cudaGetErrorString(e));

  const size_t fast_smem = kSharedHeader + (size_t)kFastCap * 8;
  const int gen_blocks = (int)(rows < 148 ? rows : 148);
  int rc;
  if (dtype == TLX_BF16) {
    const size_t gen_smem = kSharedHeader + (size_t)kWindow * 4;
    if ((rc = ensure_smem((const void*)sample_fast_kernel<TLX_BF16>, fast_smem, "sample")) != TLX_OK) return rc;
    if ((rc = ensure_smem((const void*)sample_general_bf16_kernel, gen_smem, "sample")) != TLX_OK) return rc;
    sample_fast_kernel<TLX_BF16><<<(unsigned)rows, kFastThreads, fast_smem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (fast kernel)");
    sample_general_bf16_kernel<<<gen_blocks, kGenThreads, gen_smem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (general kernel)");
  } else {
    const size_t gen_smem = kSharedHeader + (size_t)kHistBins * 8;
    if ((rc = ensure_smem((const void*)sample_fast_kernel<TLX_F32>, fast_smem, "sample")) != TLX_OK) return rc;
    if ((rc = ensure_smem((const void*)sample_general_radix_kernel<TLX_F32>, gen_smem, "sample")) != TLX_OK) return rc;
    sample_fast_kernel<TLX_F32><<<(unsigned)rows, kFastThreads, fast_smem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (fast kernel)");
    sample_general_radix_kernel<TLX_F32><<<gen_blocks, kGenThreads, gen_smem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (general kernel)");
  }
  return TLX_OK;
}

int tlx_top_p_and_sample(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx, int64_t rows,
                         int k, const float* top_p, const float* temperature, const float* noise,
                         int64_t noise_stride, uint32_t key0, uint32_t key1, int64_t vocab_size, double replace_val,
                         int64_t dim0_offset, int32_t* out_tokens) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && k >= 1, "top_p_and_sample: bad extent");
  if (k > 1024) return set_error(TLX_ERR_UNSUPPORTED, "top_p_and_sample: k=%d exceeds 1024", k);
  TLX_CHECK_ARG(vocab_size >= 1, "top_p_and_sample: vocab_size must be positive");
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(topk_logits && topk_idx && top_p && temperature && out_tokens, "top_p_and_sample: null pointer");
  NoiseSrc ns{noise, noise_stride, key0, key1, vocab_size};
  if (dtype == TLX_F32) {
    top_p_and_sample_kernel<TLX_F32><<<(unsigned)rows, 256, 0, st>>>((const float*)topk_logits, topk_idx, k, top_p,
                                                                      temperature, ns, (float)replace_val, dim0_offset,
                                                                      out_tokens);
  } else if (dtype == TLX_BF16) {
    top_p_and_sample_kernel<TLX_BF16><<<(unsigned)rows, 256, 0, st>>>(
        (const __nv_bfloat16*)topk_logits, topk_idx, k, top_p, temperature, ns,
        __float2bfloat16_rn((float)replace_val), dim0_offset, out_tokens);
  } else {
    return set_error(TLX_ERR_UNSUPPORTED, "top_p_and_sample: dtype %d not supported (f32, bf16)", dtype);
  }
  TLX_CHECK_LAUNCH("top_p_and_sample");
  return TLX_OK;
}

int tlx_top_p_mask(void* stream, const float* topk_logits, const float* p, int k, int64_t batch, double replace_val,
                   float* out) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(k >= 1 && batch >= 0, "top_p_mask: bad extent");
  if (k > 1024) return set_error(TLX_ERR_UNSUPPORTED, "top_p_mask: k=%d exceeds 1024", k);
  if (batch == 0) return TLX_OK;
  TLX_CHECK_ARG(topk_logits && p && out, "top_p_mask: null pointer");
  top_p_mask_kernel<<<(unsigned)batch, 128, 0, st>>>(topk_logits, p, k, batch, (float)replace_val, out);
  TLX_CHECK_LAUNCH("top_p_mask");
  return TLX_OK;
}

int tlx_gumbel_argmax(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1, int64_t rows,
                      int64_t cols, uint32_t key0, uint32_t key1, int64_t dim1_size, int axis, int32_t* out_pos) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(axis == 0 || axis == 1, "gumbel_argmax: axis must be 0 or 1, got %d", axis);
  TLX_CHECK_ARG(rows > 0 && cols > 0 && dim1_size > 0, "gumbel_argmax: bad extent");
  TLX_CHECK_ARG(logits && idx0 && idx1 && out_pos, "gumbel_argmax: null pointer");
  const int64_t lines = axis == 1 ? rows : cols;
  gumbel_argmax_kernel<<<(unsigned)lines, 256, 0, st>>>(logits, idx0, idx1, rows, cols, key0, key1, dim1_size, axis,
                                                       out_pos);
  TLX_CHECK_LAUNCH("gumbel_argmax");
  return TLX_OK;
}

int tlx_merge_and_sample(void* stream, const float* cand_vals, const int32_t* cand_idx, const float* cand_noise,
                         int64_t rows, int n_cand, int k_per_block, int64_t block_stride, int64_t row_stride,
                         const int32_t* top_k, const float* top_p, const float* temperature, int32_t* out_tokens) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && n_cand >= 1, "merge_and_sample: bad extent");
  TLX_CHECK_ARG(k_per_block >= 1 && n_cand % k_per_block == 0, "merge_and_sample: n_cand must be a multiple of k_per_block");
  TLX_CHECK_ARG(row_stride >= k_per_block && block_stride >= 0, "merge_and_sample: bad strides");
  if (n_cand > kMergeMaxCand)
    return set_error(TLX_ERR_UNSUPPORTED, "merge_and_sample: %d candidates exceed %d", n_cand, kMergeMaxCand);
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(cand_vals && cand_idx && cand_noise && top_k && top_p && temperature && out_tokens,
                "merge_and_sample: null pointer");
  int P = 2;
  while (P < n_cand) P <<= 1;
  const size_t smem = kSharedHeader + (size_t)P * 8;
  int rc;
  if ((rc = ensure_smem((const void*)merge_and_sample_kernel, smem, "merge_and_sample")) != TLX_OK) return rc;
  merge_and_sample_kernel<<<(unsigned)rows, kMergeThreads, smem, st>>>(
      cand_vals, cand_idx, cand_noise, n_cand, k_per_block, block_stride, row_stride, top_k, top_p, temperature, out_tokens);
  TLX_CHECK_LAUNCH("merge_and_sample");
  return TLX_OK;
}

}  // extern "C"
