// Row-wise exact / single-pass top-k and the per-shard candidate stage of the
// vocab-sharded sampler.  One CTA per row: the streaming collector leaves a superset of
// the top-k in shared memory, a bitonic network orders it by (value desc, index asc).
#include "select.cuh"
#include "exchange.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace tlx {

constexpr int kTopkThreads = 512;

struct TopkParams {
  const void* x;
  int64_t rows, n, row_stride;
  int k_max;
  const int32_t* k_per_row;
  int use_replace;
  double replace_val;
  int mode;
  void* out_vals;
  int32_t* out_idx;
  int32_t* out_valid;
  int32_t* out_depths;
  void* out_cutoff;
  // candidate stage of the vocab-sharded sampler (all null / zero for plain top-k)
  float* cand_vals;
  int32_t* cand_idx;
  float* cand_noise;
  int64_t col_offset;
  int64_t dim0_offset;
  NoiseSrc noise;
  ExchangeTargets ex;   // ex.world > 0: the candidates go to every rank's exchange buffer instead
};

template <int DT>
__device__ __forceinline__ typename Elem<DT>::type cast_replace(double v) {
  if constexpr (DT == TLX_F32) return (float)v;
  else if constexpr (DT == TLX_BF16) return __float2bfloat16_rn((float)v);
  else if constexpr (DT == TLX_F16) return __float2half_rn((float)v);
  else if constexpr (DT == TLX_I32) return (int32_t)v;
  else return (uint32_t)v;
}

// Writes a row's results from its sorted candidate list (m valid entries, the first K are the answer).
template <int DT>
__device__ __forceinline__ void emit_row(const TopkParams& p, int64_t r, const typename Elem<DT>::type* __restrict__ row,
                                         const uint64_t* cand, int m, const SelectShared& s) {
  using T = typename Elem<DT>::type;
  const int K = p.k_max;
  const int k_row = p.k_per_row ? p.k_per_row[r] : K;
  uint32_t par = 0;   // which of the exchange buffer's two sets this step uses
  bool deliver = p.ex.world > 0;
  if (p.ex.world > 0) {
    // a call whose extents are not the buffer's stores nothing anywhere and leaves a mark
    volatile ExchangeHeader* h = reinterpret_cast<volatile ExchangeHeader*>(p.ex.peer[p.ex.rank]);
    par = h->step & 1u;
    deliver = h->rows == (uint32_t)p.rows && h->k_cand == (uint32_t)K && h->world == (uint32_t)p.ex.world;
    if (!deliver && threadIdx.x == 0) h->error = 2u;
  }
  for (int j = threadIdx.x; j < K; j += blockDim.x) {
    const uint64_t c = cand[j];
    const int32_t col = (int32_t)cand_low(c);
    const bool have = j < m;
    if (p.cand_vals || p.ex.world > 0) {
      // candidate stage: f32 value, global token id, noise at that token
      const float v = have ? elem_as_float<DT>(row[col]) : -INFINITY;
      const int64_t tok = (int64_t)col + p.col_offset;
      float u = 0.5f;
      if (have) u = p.noise.dense ? __ldg(p.noise.dense + r * p.noise.stride + col) : p.noise.at(r + p.dim0_offset, tok);
      if (p.ex.world > 0) {
        if (!deliver) continue;
        // slot `rank` of every rank's buffer, this rank's own included, starting with the next rank
        const size_t plane = (size_t)p.rows * K;
        for (int i = 0; i < p.ex.world; ++i) {
          int peer = p.ex.rank + 1 + i;
          if (peer >= p.ex.world) peer -= p.ex.world;
          float* blk = reinterpret_cast<float*>(p.ex.peer[peer] + p.ex.off_cand[par]) + (size_t)p.ex.rank * 3 * plane;
          blk[r * K + j] = v;
          reinterpret_cast<int32_t*>(blk)[plane + r * K + j] = have ? (int32_t)tok : -1;
          blk[2 * plane + r * K + j] = u;
        }
      } else {
        p.cand_vals[r * K + j] = v;
        p.cand_idx[r * K + j] = have ? (int32_t)tok : -1;
        p.cand_noise[r * K + j] = u;
      }
    } else {
      T v = have ? row[col] : cast_replace<DT>(0.0);
      if (p.use_replace && j >= k_row) v = cast_replace<DT>(p.replace_val);
      reinterpret_cast<T*>(p.out_vals)[r * K + j] = v;
      p.out_idx[r * K + j] = have ? col : 0;
    }
  }
  if (p.ex.world > 0) {
    // the row's block is on its way to every rank: one arrival count each, released after the stores
    __syncthreads();
    if (deliver && (int)threadIdx.x < p.ex.world) {
      __threadfence_system();
      atomicAdd_system(reinterpret_cast<uint32_t*>(p.ex.peer[threadIdx.x] + p.ex.off_flags[par]) + r, 1u);
    }
  }
  if (threadIdx.x == 0) {
    if (p.out_depths) p.out_depths[r] = s.refinements;
    if (p.out_cutoff) {
      if constexpr (DT == TLX_I32 || DT == TLX_U32)
        reinterpret_cast<int32_t*>(p.out_cutoff)[r] = (int32_t)Elem<TLX_I32>::from_key((uint32_t)s.bin << kHistShift);
      else
        reinterpret_cast<float*>(p.out_cutoff)[r] = bin_lower_value(s.bin);
    }
  }
}

template <int DT, int CAP>
__global__ void __launch_bounds__(kTopkThreads) topk_kernel(TopkParams p) {
  using T = typename Elem<DT>::type;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  const int64_t r = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(p.x) + r * p.row_stride;
  const int K = p.k_max;
  // exchange mode: the merge kernel that follows waits for the rows' arrival counts, not for this kernel
  if (p.ex.world > 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  bool ok = collect_row<DT, CAP>(row, p.n, K, s, cand);
  if (!ok) {
    if (p.mode == 0) {
      exact_select_row<DT>(row, p.n, K, s, cand);
    } else {
      if (threadIdx.x == 0) { if (p.out_valid) atomicExch(p.out_valid, 0); s.fill = CAP; }
      __syncthreads();
    }
  }
  const int m = min(s.fill, CAP);
  sort_candidates(cand, m);

  emit_row<DT>(p, r, row, cand, m, s);
}

// ---- many short rows ---------------------------------------------------------------------------------
// A CTA of 128 threads per row, eight of them per SM, two passes over the row (the second one finds the
// row in L2).  Pass 1 keeps, per thread, the running maximum of every slot of its 16-byte vectors: 128 x
// kSlots group maxima, each an element of the row.  The K-th largest of them (K <= number of groups) is
// a lower bound of the row's K-th largest element, and with groups of a few dozen elements it is a tight
// one: for K = 50 of 19 000 elements about K + 1 elements lie at or above it.  Pass 2 collects those, a
// bitonic network orders them.  The bound is taken on the top 16 key bits.  NaNs have the greatest key:
// the maxima skip them (so they stay elements of the row), pass 2 admits them by its negated compare.
constexpr int kShortThreads = 128;
constexpr int kShortCap = 1024;
constexpr int kShortMaxK = 128;

template <int DT> struct GroupMax;
template <> struct GroupMax<TLX_BF16> {
  static constexpr int kSlots = 8;
  __nv_bfloat162 m[4];
  __device__ __forceinline__ void init() {
    const __nv_bfloat16 ninf = __float2bfloat16_rn(-INFINITY);
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = __halves2bfloat162(ninf, ninf);
  }
  __device__ __forceinline__ void add(const uint4& v) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = __hmax2(m[j], e[j]);
  }
  __device__ __forceinline__ void add_one(__nv_bfloat16 x) { m[0] = __hmax2(m[0], __halves2bfloat162(x, m[0].y)); }
  __device__ __forceinline__ float slot(int j) const {
    return (j & 1) ? __high2float(m[j >> 1]) : __low2float(m[j >> 1]);
  }
};
template <> struct GroupMax<TLX_F16> {
  static constexpr int kSlots = 8;
  __half2 m[4];
  __device__ __forceinline__ void init() {
    const __half ninf = __float2half_rn(-INFINITY);
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = __halves2half2(ninf, ninf);
  }
  __device__ __forceinline__ void add(const uint4& v) {
    const __half2* e = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = __hmax2(m[j], e[j]);
  }
  __device__ __forceinline__ void add_one(__half x) { m[0] = __hmax2(m[0], __halves2half2(x, __high2half(m[0]))); }
  __device__ __forceinline__ float slot(int j) const {
    return (j & 1) ? __high2float(m[j >> 1]) : __low2float(m[j >> 1]);
  }
};
template <> struct GroupMax<TLX_F32> {
  static constexpr int kSlots = 4;
  float m[4];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = -INFINITY;
  }
  __device__ __forceinline__ void add(const uint4& v) {
    const float* e = reinterpret_cast<const float*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) m[j] = fmaxf(m[j], e[j]);
  }
  __device__ __forceinline__ void add_one(float x) { m[0] = fmaxf(m[0], x); }
  __device__ __forceinline__ float slot(int j) const { return m[j]; }
};

// Row traversal by 16-byte vectors: fv(vector, first column) in the aligned body, kU loads in flight per
// thread; fs(element, column) for the unaligned head and tail.  sub > 1 visits only every sub-th run of
// blockDim vectors (a sample of the row in contiguous 2 KB pieces).
template <int DT, int kU, typename FV, typename FS>
__device__ __forceinline__ void for_each_vec(const typename Elem<DT>::type* __restrict__ row, int64_t n, int sub, FV&& fv,
                                             FS&& fs) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  const uintptr_t addr = reinterpret_cast<uintptr_t>(row);
  int64_t head = (int64_t)(((16 - (addr & 15)) & 15) / sizeof(T));
  if (head > n) head = n;
  for (int64_t c = threadIdx.x; c < head; c += blockDim.x) fs(row[c], c);
  const int64_t nvec = (n - head) / VEC;
  const uint4* vp = reinterpret_cast<const uint4*>(row + head);
  const int64_t step = (int64_t)blockDim.x * sub;
  int64_t i = threadIdx.x;
  for (; i + (int64_t)(kU - 1) * step < nvec; i += (int64_t)kU * step) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) v[u] = __ldg(vp + i + (int64_t)u * step);
#pragma unroll
    for (int u = 0; u < kU; ++u) fv(v[u], head + (i + (int64_t)u * step) * VEC);
  }
#pragma unroll 1
  for (; i < nvec; i += step) fv(__ldg(vp + i), head + i * VEC);
#pragma unroll 1
  for (int64_t c = head + nvec * VEC + threadIdx.x; c < n; c += blockDim.x) fs(row[c], c);
}

// The elements of one vector that lie at or above the bound join the candidate list.
template <int DT>
static __device__ __noinline__ void push_vector(uint4 v, int64_t cb, uint32_t t16, float thr, int* fill, uint64_t* cand,
                                            int cap) {
  using T = typename Elem<DT>::type;
  const T* x = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int j = 0; j < 16 / (int)sizeof(T); ++j) {
    if (!(elem_as_float<DT>(x[j]) < thr)) {
      const uint32_t key = Elem<DT>::key(x[j]);
      if ((key >> 16) >= t16) {
        const int slot = atomicAdd(fill, 1);
        if (slot < cap) cand[slot] = cand_make(key, (uint32_t)(cb + j));
      }
    }
  }
}

// The K-th largest of the G 16-bit keys in shared memory (1 <= K <= G): two counting passes of 8 bits.
// hist: 512 words (one histogram per pass), pick: 4 words, both in shared memory.  All threads call.  The
// bin that holds the `need`-th largest is found by warp 0 alone (eight bins per lane, one shuffle scan):
// five CTA barriers in all.
__device__ __forceinline__ void warp_pick_bin(const uint32_t* h, int need, int* out) {
  const int lane = lane_id();
  const int hi = 255 - 8 * lane;   // lane l owns bins hi, hi-1, ..., hi-7 (descending)
  uint32_t local = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) local += h[hi - j];
  uint32_t incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += up;
  }
  const uint32_t excl = incl - local;
  if (excl < (uint32_t)need && incl >= (uint32_t)need) {
    uint32_t run = excl;
    for (int j = 0; j < 8; ++j) {
      const uint32_t c = h[hi - j];
      if (run + c >= (uint32_t)need) { out[0] = hi - j; out[1] = (int)run; break; }
      run += c;
    }
  }
}

static __device__ __noinline__ uint32_t kth_largest_u16(const uint16_t* keys, int G, int K, uint32_t* hist, int* pick) {
  for (int i = threadIdx.x; i < 512; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < G; i += blockDim.x) atomicAdd(&hist[keys[i] >> 8], 1u);
  __syncthreads();
  if (warp_id() == 0) warp_pick_bin(hist, K, pick);
  __syncthreads();
  const uint32_t top = (uint32_t)pick[0];
  const int need = K - pick[1];
  for (int i = threadIdx.x; i < G; i += blockDim.x) {
    const uint32_t k = keys[i];
    if ((k >> 8) == top) atomicAdd(&hist[256 + (k & 255u)], 1u);
  }
  __syncthreads();
  if (warp_id() == 0) warp_pick_bin(hist + 256, need, pick + 2);
  __syncthreads();
  return (top << 8) | (uint32_t)pick[2];
}

template <int DT>
__global__ void __launch_bounds__(kShortThreads, 8) topk_short_kernel(TopkParams p) {
  using T = typename Elem<DT>::type;
  constexpr int kSlots = GroupMax<DT>::kSlots;
  constexpr int G = kShortThreads * kSlots;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  // the group keys and the small histogram live in the big histogram's space, which only the fallback uses
  uint16_t* gkeys = reinterpret_cast<uint16_t*>(s.hist);            // G * 2 bytes <= 2 KB
  uint32_t* hist8 = s.hist + 1024;                                    // 512 words
  const int64_t r = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(p.x) + r * p.row_stride;
  const int K = p.k_max;
  const int64_t n = p.n;
  // exchange mode: the merge kernel that follows waits for the rows' arrival counts, not for this kernel
  if (p.ex.world > 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // rows that L2 would not keep between the passes give their bound from a quarter of the row
  const int sub = n * (int64_t)sizeof(T) > (128 << 10) ? 4 : 1;
  // bf16 rows of up to 4096 vectors (64 KB) read in full by pass 1: pass 1 also leaves every vector's greatest
  // element (NaN if it holds one) in shared memory, in the candidate list's space, and pass 2 reads those
  // 2 bytes per vector instead of the row
  constexpr int VEC = 16 / (int)sizeof(T);
  int64_t head = (int64_t)(((16 - (reinterpret_cast<uintptr_t>(row) & 15)) & 15) / sizeof(T));
  if (head > n) head = n;
  const int64_t nvec = (n - head) / VEC;
  bool vec_maxima = false;
  if constexpr (DT == TLX_BF16) vec_maxima = sub == 1 && nvec <= kShortCap * 4;
  __nv_bfloat16* vmax = reinterpret_cast<__nv_bfloat16*>(cand);
  GroupMax<DT> gm;
  gm.init();
  if constexpr (DT == TLX_BF16) {
    if (vec_maxima) {
      const __nv_bfloat16 ninf = __float2bfloat16_rn(-INFINITY);
      for (int64_t i = nvec + threadIdx.x; i < ((nvec + 7) & ~(int64_t)7); i += blockDim.x) vmax[i] = ninf;
      for_each_vec<DT, 10>(row, n, 1,
        [&](const uint4& v, int64_t cb) {
          gm.add(v);
          const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&v);
          const __nv_bfloat162 a = __hmax2_nan(__hmax2_nan(e[0], e[1]), __hmax2_nan(e[2], e[3]));
          vmax[(cb - head) >> 3] = __hmax_nan(__low2bfloat16(a), __high2bfloat16(a));
        },
        [&](T x, int64_t) { gm.add_one(x); });
    }
  }
  if (!vec_maxima)
    for_each_vec<DT, 10>(row, n, sub, [&](const uint4& v, int64_t) { gm.add(v); }, [&](T x, int64_t) { gm.add_one(x); });
#pragma unroll
  for (int j = 0; j < kSlots; ++j) gkeys[threadIdx.x * kSlots + j] = (uint16_t)(f32_key(gm.slot(j)) >> 16);
  if (threadIdx.x == 0) { s.fill = 0; s.bin = 0; s.above = 0; s.refinements = 0; }
  __syncthreads();
  const uint32_t t16 = kth_largest_u16(gkeys, G, K, hist8, s.tmp_i);
  // lower edge of the bound's 16-bit bin as a value; a NaN pattern (the bin of -inf) admits everything
  const float thr = key_f32(t16 << 16);

  auto push_one = [&](T x, int64_t c) {
    if (!(elem_as_float<DT>(x) < thr)) {
      const uint32_t key = Elem<DT>::key(x);
      if ((key >> 16) >= t16) {
        const int slot = atomicAdd(&s.fill, 1);
        if (slot < kShortCap) cand[slot] = cand_make(key, (uint32_t)c);
      }
    }
  };
  // The streaming loop only notes which vectors hold an element at or above the bound (about one per
  // candidate); the noted vectors are then read again, one per thread, and their elements pushed.
  uint32_t* noted = s.hist + 2048;          // up to kShortCap first columns, in the fallback's histogram space
  int* nnoted = &s.above;                   // (tmp_i holds the bound's picks, which threads may still be reading)
  if (threadIdx.x == 0) *nnoted = 0;
  __syncthreads();
  auto note = [&](int64_t cb) {
    const int slot = atomicAdd(nnoted, 1);
    if (slot < kShortCap) noted[slot] = (uint32_t)cb;
  };
  if constexpr (DT == TLX_BF16) {
    const __nv_bfloat16 tb = __ushort_as_bfloat16((unsigned short)(__float_as_uint(thr) >> 16));
    const __nv_bfloat162 t2 = __halves2bfloat162(tb, tb);
    if (vec_maxima) {
      // eight vectors' maxima per 16-byte load; the few elements before and after the aligned body are
      // pushed after the barrier below (the candidate list shares its space with the maxima)
      const uint4* vm4 = reinterpret_cast<const uint4*>(vmax);
      const int groups = (int)((nvec + 7) >> 3);
      for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        const uint4 w = vm4[g];
        const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&w);
        if (!(__hblt2(e[0], t2) && __hblt2(e[1], t2) && __hblt2(e[2], t2) && __hblt2(e[3], t2))) {
          const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(&w);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (g * 8 + j < nvec && !__hlt(x[j], tb)) note(head + ((int64_t)g * 8 + j) * VEC);   // not the padding
        }
      }
    } else {
      for_each_vec<DT, 10>(row, n, 1,
        [&](const uint4& v, int64_t cb) {
          const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&v);
          // __hblt2: both halves less than the bound (false when either is a NaN)
          if (!(__hblt2(e[0], t2) && __hblt2(e[1], t2) && __hblt2(e[2], t2) && __hblt2(e[3], t2))) note(cb);
        },
        push_one);
    }
  } else if constexpr (DT == TLX_F16) {
    for_each_vec<DT, 10>(row, n, 1,
      [&](const uint4& v, int64_t cb) {
        const __half2* e = reinterpret_cast<const __half2*>(&v);
        bool any = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(e[j]);
          any = any || !(f.x < thr) || !(f.y < thr);
        }
        if (any) note(cb);
      },
      push_one);
  } else {
    for_each_vec<DT, 10>(row, n, 1,
      [&](const uint4& v, int64_t cb) {
        const float* e = reinterpret_cast<const float*>(&v);
        if (!(e[0] < thr) || !(e[1] < thr) || !(e[2] < thr) || !(e[3] < thr)) note(cb);
      },
      push_one);
  }
  __syncthreads();
  if (vec_maxima) {
    for (int64_t c = threadIdx.x; c < head; c += blockDim.x) push_one(row[c], c);
    for (int64_t c = head + nvec * VEC + threadIdx.x; c < n; c += blockDim.x) push_one(row[c], c);
  }
  if (*nnoted > kShortCap) {
    if (threadIdx.x == 0) s.fill = kShortCap + 1;   // more vectors than the list holds: the exact fallback
  } else {
    for (int l = threadIdx.x; l < *nnoted; l += blockDim.x) {
      const int64_t cb = noted[l];
      push_vector<DT>(__ldg(reinterpret_cast<const uint4*>(row + cb)), cb, t16, thr, &s.fill, cand, kShortCap);
    }
  }
  __syncthreads();
  if (s.fill > kShortCap) exact_select_row<DT>(row, n, K, s, cand);   // huge groups of equal values
  const int m = min(s.fill, kShortCap);
  if (m <= 96) {
    // a handful of candidates: every thread counts the composites below its own (they are distinct) and
    // puts it at that place; no network, no barriers in between
    uint64_t* placed = reinterpret_cast<uint64_t*>(s.hist + 2048);   // 96 slots in the fallback's histogram space
    if ((int)threadIdx.x < m) {
      const uint64_t c = cand[threadIdx.x];
      int below = 0;
      for (int i = 0; i < m; ++i) below += cand[i] < c ? 1 : 0;
      placed[below] = c;
    }
    __syncthreads();
    emit_row<DT>(p, r, row, placed, m, s);
  } else {
    sort_candidates(cand, m);
    emit_row<DT>(p, r, row, cand, m, s);
  }
}

// Whether the two-pass kernel serves a call: floating-point rows, K <= 128, exact mode without the
// diagnostics of the one-pass kernel, and enough rows to fill the eight CTAs per SM.
static bool short_rows_apply(int dtype, const TopkParams& p) {
  static const char* force = getenv("TLX_TOPK_PATH");   // "short" / "long": comparison runs
  if (dtype != TLX_F32 && dtype != TLX_BF16 && dtype != TLX_F16) return false;
  if (p.k_max > kShortMaxK || p.mode != 0 || p.out_valid || p.out_depths || p.out_cutoff) return false;
  if (force && !strcmp(force, "short")) return true;
  if (force && !strcmp(force, "long")) return false;
  return p.rows >= 256 && p.n >= 2048;
}

template <int DT>
static int launch_topk_short(cudaStream_t st, const TopkParams& p) {
  const size_t smem = ((sizeof(SelectShared) + 15) & ~size_t(15)) + (size_t)kShortCap * 8;
  // eight CTAs of 25 KB per SM need the large shared-memory configuration: asked for once per device
  static std::mutex mu;
  static bool asked[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !asked[dev]) {
      cudaError_t e = cudaFuncSetAttribute(topk_short_kernel<DT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           (int)cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "top_k: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      if (dev >= 0 && dev < 64) asked[dev] = true;
    }
  }
  topk_short_kernel<DT><<<(unsigned)p.rows, kShortThreads, smem, st>>>(p);
  TLX_CHECK_LAUNCH("top_k (short rows)");
  return TLX_OK;
}

template <int DT, int CAP>
static int launch_topk_cap(cudaStream_t st, const TopkParams& p) {
  const size_t smem = ((sizeof(SelectShared) + 15) & ~size_t(15)) + (size_t)CAP * 8;
  // the shared-memory limit of this instantiation is raised once per device, not per call
  static std::mutex mu;
  static bool raised[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !raised[dev]) {
      cudaError_t e = cudaFuncSetAttribute(topk_kernel<DT, CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "top_k: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      if (dev >= 0 && dev < 64) raised[dev] = true;
    }
  }
  // out_valid starts as 1: a stream-ordered 4-byte copy node instead of a kernel of its own
  if (p.out_valid) {
    static const int32_t one = 1;
    cudaError_t e = cudaMemcpyAsync(p.out_valid, &one, sizeof(one), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "top_k: cudaMemcpyAsync: %s", cudaGetErrorString(e));
  }
  topk_kernel<DT, CAP><<<(unsigned)p.rows, kTopkThreads, smem, st>>>(p);
  TLX_CHECK_LAUNCH("top_k");
  return TLX_OK;
}

template <int DT>
static int launch_topk(cudaStream_t st, const TopkParams& p) {
  if (p.k_max <= 256) return launch_topk_cap<DT, 1024>(st, p);
  if (p.k_max <= 1024) return launch_topk_cap<DT, 4096>(st, p);
  return launch_topk_cap<DT, 8192>(st, p);
}

static int dispatch_topk(cudaStream_t st, int dtype, const TopkParams& p, const char* what) {
  if (short_rows_apply(dtype, p)) {
    switch (dtype) {
      case TLX_F32: return launch_topk_short<TLX_F32>(st, p);
      case TLX_BF16: return launch_topk_short<TLX_BF16>(st, p);
      default: return launch_topk_short<TLX_F16>(st, p);
    }
  }
  switch (dtype) {
    case TLX_F32: return launch_topk<TLX_F32>(st, p);
    case TLX_BF16: return launch_topk<TLX_BF16>(st, p);
    case TLX_F16: return launch_topk<TLX_F16>(st, p);
    case TLX_I32: return launch_topk<TLX_I32>(st, p);
    case TLX_U32: return launch_topk<TLX_U32>(st, p);
    default: return set_error(TLX_ERR_UNSUPPORTED, "%s: dtype %d not supported", what, dtype);
  }
}

// ---- a handful of long rows: every row is cut into parts, each part's top-k is found by a CTA of its own
// (the same kernel on rows * parts "rows"), and a second pass takes the top-k of the parts' candidates.
// Among equal values the parts' order and, inside a part, the ascending index order of its candidates keep
// the lower original index first, as the one-pass kernel does.
struct SplitPlan {
  int parts = 0;          // 0: no split
  int64_t part_len = 0;
  size_t off_idx_a = 0, off_idx_b = 0, bytes = 0;
};

static SplitPlan split_plan(int64_t rows, int64_t n, int k_max, int elem_bytes) {
  SplitPlan sp;
  if (rows <= 0 || rows > 16 || n < 16384 || k_max > 256) return sp;   // more rows fill the GPU by themselves
  for (int parts = 16; parts >= 4; parts >>= 1) {
    if (n % parts) continue;
    const int64_t len = n / parts;
    if (len < 2048 || len < 4 * (int64_t)k_max || (len * elem_bytes) % 16) continue;
    sp.parts = parts;
    sp.part_len = len;
    break;
  }
  if (!sp.parts) return sp;
  auto align = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t cand = (size_t)rows * sp.parts * k_max;
  sp.off_idx_a = align(cand * elem_bytes);
  sp.off_idx_b = sp.off_idx_a + align(cand * 4);
  sp.bytes = sp.off_idx_b + align((size_t)rows * k_max * 4);
  return sp;
}

// out_idx[r, j] = original column of the candidate that the second pass picked at position pos_b[r, j]
__global__ void topk_map_index_kernel(const int32_t* __restrict__ idx_a, const int32_t* __restrict__ pos_b,
                                      int32_t* __restrict__ out_idx, int64_t rows, int k, int parts, int64_t part_len) {
  const int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (e >= rows * k) return;
  const int64_t r = e / k;
  const int pos = pos_b[e];
  out_idx[e] = idx_a[r * (int64_t)parts * k + pos] + (int32_t)((pos / k) * part_len);
}

}  // namespace tlx

using namespace tlx;

extern "C" {

size_t tlx_top_k_workspace_bytes(int64_t rows, int64_t n, int k_max) { return split_plan(rows, n, k_max, 4).bytes; }

int tlx_top_k(void* stream, const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int k_max,
              const int32_t* k_per_row, int use_replace, double replace_val, int mode, void* out_vals,
              int32_t* out_idx, int32_t* out_valid, int32_t* out_depths, void* out_cutoff, void* workspace,
              size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && n >= 0, "top_k: negative extent");
  TLX_CHECK_ARG(k_max >= 1, "top_k: k must be >= 1, got %d", k_max);
  if (k_max > TLX_TOPK_MAX_K)
    return set_error(TLX_ERR_UNSUPPORTED, "top_k: k=%d exceeds the supported maximum %d", k_max, TLX_TOPK_MAX_K);
  TLX_CHECK_ARG((int64_t)k_max <= n, "top_k: k=%d exceeds the row length %lld", k_max, (long long)n);
  TLX_CHECK_ARG(mode == 0 || mode == 1, "top_k: mode must be 0 or 1");
  TLX_CHECK_ARG(n < (1ll << 31) && rows < (1ll << 31), "top_k: extent too large");
  TLX_CHECK_ARG(row_stride >= n, "top_k: row stride smaller than the row");
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(x && out_vals && out_idx, "top_k: null pointer");
  // few long rows, exact mode, no diagnostics asked for, and scratch given: split the rows over CTAs
  const int es = dtype == TLX_BF16 || dtype == TLX_F16 ? 2 : 4;
  const SplitPlan sp = split_plan(rows, n, k_max, es);
  if (sp.parts && mode == 0 && !out_valid && !out_depths && !out_cutoff && row_stride == n && workspace &&
      workspace_bytes >= sp.bytes && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    unsigned char* ws = (unsigned char*)workspace;
    TopkParams a{};
    a.x = x; a.rows = rows * sp.parts; a.n = sp.part_len; a.row_stride = sp.part_len; a.k_max = k_max;
    a.out_vals = ws; a.out_idx = (int32_t*)(ws + sp.off_idx_a);
    int rc = dispatch_topk(st, dtype, a, "top_k");
    if (rc != TLX_OK) return rc;
    TopkParams b{};
    b.x = ws; b.rows = rows; b.n = (int64_t)sp.parts * k_max; b.row_stride = b.n; b.k_max = k_max;
    b.k_per_row = k_per_row; b.use_replace = use_replace; b.replace_val = replace_val;
    b.out_vals = out_vals; b.out_idx = (int32_t*)(ws + sp.off_idx_b);
    if ((rc = dispatch_topk(st, dtype, b, "top_k")) != TLX_OK) return rc;
    const int64_t total = rows * k_max;
    topk_map_index_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const int32_t*)(ws + sp.off_idx_a),
                                                                          (const int32_t*)(ws + sp.off_idx_b), out_idx, rows,
                                                                          k_max, sp.parts, sp.part_len);
    TLX_CHECK_LAUNCH("top_k (index map)");
    return TLX_OK;
  }
  TopkParams p{};
  p.x = x; p.rows = rows; p.n = n; p.row_stride = row_stride; p.k_max = k_max; p.k_per_row = k_per_row;
  p.use_replace = use_replace; p.replace_val = replace_val; p.mode = mode; p.out_vals = out_vals;
  p.out_idx = out_idx; p.out_valid = out_valid; p.out_depths = out_depths; p.out_cutoff = out_cutoff;
  return dispatch_topk(st, dtype, p, "top_k");
}

size_t tlx_shard_candidates_workspace_bytes(int64_t, int64_t, int) { return 0; }

static int shard_candidates_impl(void* stream, const void* logits, int dtype, int64_t rows, int64_t v_local,
                                 int64_t row_stride, int64_t col_offset, int k_cand, const float* noise,
                                 int64_t noise_stride, uint32_t key0, uint32_t key1, const uint32_t* key_dev,
                                 int64_t vocab_total, int64_t dim0_offset, const int32_t* dim0_offset_dev,
                                 float* out_vals, int32_t* out_idx, float* out_noise,
                                 const ExchangeTargets* ex = nullptr) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && v_local > 0, "shard_candidates: bad extent");
  TLX_CHECK_ARG(k_cand >= 1 && k_cand <= 1024, "shard_candidates: k_cand must be in [1, 1024], got %d", k_cand);
  TLX_CHECK_ARG((int64_t)k_cand <= v_local, "shard_candidates: k_cand exceeds the shard width");
  TLX_CHECK_ARG(dtype == TLX_F32 || dtype == TLX_BF16 || dtype == TLX_F16, "shard_candidates: float logits only");
  TLX_CHECK_ARG(row_stride >= v_local, "shard_candidates: row stride smaller than the row");
  TLX_CHECK_ARG(col_offset >= 0 && col_offset + v_local <= (1ll << 31), "shard_candidates: token ids exceed int32");
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(logits && (ex || (out_vals && out_idx && out_noise)), "shard_candidates: null pointer");
  TopkParams p{};
  if (ex) p.ex = *ex;
  p.x = logits; p.rows = rows; p.n = v_local; p.row_stride = row_stride; p.k_max = k_cand;
  p.cand_vals = out_vals; p.cand_idx = out_idx; p.cand_noise = out_noise; p.col_offset = col_offset;
  p.dim0_offset = dim0_offset;
  p.noise.dense = noise; p.noise.stride = noise_stride; p.noise.k0 = key0; p.noise.k1 = key1; p.noise.vocab = vocab_total;
  p.noise.key_dev = key_dev; p.noise.row_offset_dev = dim0_offset_dev;
  return dispatch_topk(st, dtype, p, "shard_candidates");
}

int tlx_shard_candidates(void* stream, const void* logits, int dtype, int64_t rows, int64_t v_local,
                         int64_t row_stride, int64_t col_offset, int k_cand, const float* noise, int64_t noise_stride,
                         uint32_t key0, uint32_t key1, int64_t vocab_total, int64_t dim0_offset, float* out_vals,
                         int32_t* out_idx, float* out_noise, void*, size_t) {
  return shard_candidates_impl(stream, logits, dtype, rows, v_local, row_stride, col_offset, k_cand, noise, noise_stride,
                               key0, key1, nullptr, vocab_total, dim0_offset, nullptr, out_vals, out_idx, out_noise);
}

int tlx_shard_candidates_dev(void* stream, const void* logits, int dtype, int64_t rows, int64_t v_local,
                             int64_t row_stride, int64_t col_offset, int k_cand, const float* noise,
                             int64_t noise_stride, const uint32_t* key_dev, int64_t vocab_total,
                             const int32_t* dim0_offset_dev, float* out_vals, int32_t* out_idx, float* out_noise,
                             void*, size_t) {
  if (!noise && !key_dev) return set_error(TLX_ERR_INVALID, "shard_candidates: neither noise nor a key given");
  return shard_candidates_impl(stream, logits, dtype, rows, v_local, row_stride, col_offset, k_cand, noise, noise_stride,
                               0u, 0u, key_dev, vocab_total, 0, dim0_offset_dev, out_vals, out_idx, out_noise);
}

int tlx_exchange_shard_candidates(void* stream, const void* logits, int dtype, int64_t rows, int64_t v_local,
                                  int64_t row_stride, int64_t col_offset, int k_cand, const float* noise,
                                  int64_t noise_stride, const uint32_t* key_dev, uint32_t key0, uint32_t key1,
                                  int64_t vocab_total, int64_t dim0_offset, const int32_t* dim0_offset_dev, int rank,
                                  int world, void* const* exchange_of_rank) {
  TLX_CHECK_ARG(world >= 1 && world <= kExchangeMaxWorld && rank >= 0 && rank < world,
                "exchange_shard_candidates: rank %d of %d", rank, world);
  TLX_CHECK_ARG(exchange_of_rank && rows >= 1 && k_cand >= 1, "exchange_shard_candidates: bad argument");
  ExchangeTargets ex{};
  ex.world = world;
  ex.rank = rank;
  const ExchangeLayout l = exchange_layout(rows, k_cand, world);
  for (int q = 0; q < 2; ++q) { ex.off_flags[q] = l.off_flags[q]; ex.off_cand[q] = l.off_cand[q]; }
  for (int i = 0; i < world; ++i) {
    TLX_CHECK_ARG(exchange_of_rank[i], "exchange_shard_candidates: buffer of rank %d is null", i);
    ex.peer[i] = (unsigned char*)exchange_of_rank[i];
  }
  return shard_candidates_impl(stream, logits, dtype, rows, v_local, row_stride, col_offset, k_cand, noise, noise_stride,
                               key0, key1, key_dev, vocab_total, dim0_offset, dim0_offset_dev, nullptr, nullptr, nullptr,
                               &ex);
}

}  // extern "C"
