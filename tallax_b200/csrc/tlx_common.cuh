// Shared device/host helpers for the tallax_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/tallax_b200.h"

namespace tlx {

// ---- host-side error plumbing ------------------------------------------------
int set_error(int code, const char* fmt, ...);
void count_launch();   // bumps the process-wide launch counter read by tlx_kernel_launches()

#define TLX_CHECK_ARG(cond, ...)                               \
  do {                                                         \
    if (!(cond)) return ::tlx::set_error(TLX_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define TLX_CHECK_LAUNCH(what)                                                         \
  do {                                                                                 \
    ::tlx::count_launch();                                                             \
    cudaError_t e_ = cudaGetLastError();                                               \
    if (e_ != cudaSuccess)                                                             \
      return ::tlx::set_error(TLX_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e_));    \
  } while (0)

inline int dtype_bytes(int dtype) {
  switch (dtype) {
    case TLX_F32: case TLX_I32: case TLX_U32: return 4;
    case TLX_BF16: case TLX_F16: return 2;
    default: return 0;
  }
}

constexpr float kSamplingEps = 1e-5f;        // temperature below this means greedy
constexpr float kF32Tiny = 1.17549435e-38f;  // smallest normal f32: lower clamp of the noise

// ---- order-preserving keys -----------------------------------------------------
// f32 -> u32 such that unsigned compare orders like the floats; -0 is folded onto +0
// and every NaN maps to the single greatest key.
__device__ __forceinline__ uint32_t f32_key(float x) {
  uint32_t b = __float_as_uint(x);
  if (x == 0.f) b = 0u;
  uint32_t k = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (x != x) ? 0xFFFFFFFFu : k;
}
__device__ __forceinline__ float key_f32(uint32_t k) {
  uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}
__device__ __forceinline__ uint32_t i32_key(int32_t x) { return (uint32_t)x ^ 0x80000000u; }

// Typed loads of one element as (key, f32 value) -------------------------------
template <int DT> struct Elem;
template <> struct Elem<TLX_F32> {
  using type = float;
  static constexpr int kBytes = 4;
  static __device__ __forceinline__ uint32_t key(float v) { return f32_key(v); }
  static __device__ __forceinline__ float from_key(uint32_t k) { return key_f32(k); }
};
template <> struct Elem<TLX_BF16> {
  using type = __nv_bfloat16;
  static constexpr int kBytes = 2;
  static __device__ __forceinline__ uint32_t key(__nv_bfloat16 v) { return f32_key(__bfloat162float(v)); }
  static __device__ __forceinline__ __nv_bfloat16 from_key(uint32_t k) { return __float2bfloat16_rn(key_f32(k)); }
};
template <> struct Elem<TLX_F16> {
  using type = __half;
  static constexpr int kBytes = 2;
  static __device__ __forceinline__ uint32_t key(__half v) { return f32_key(__half2float(v)); }
  static __device__ __forceinline__ __half from_key(uint32_t k) { return __float2half_rn(key_f32(k)); }
};
template <> struct Elem<TLX_I32> {
  using type = int32_t;
  static constexpr int kBytes = 4;
  static __device__ __forceinline__ uint32_t key(int32_t v) { return i32_key(v); }
  static __device__ __forceinline__ int32_t from_key(uint32_t k) { return (int32_t)(k ^ 0x80000000u); }
};
template <> struct Elem<TLX_U32> {
  using type = uint32_t;
  static constexpr int kBytes = 4;
  static __device__ __forceinline__ uint32_t key(uint32_t v) { return v; }
  static __device__ __forceinline__ uint32_t from_key(uint32_t k) { return k; }
};

// ---- warp / block collectives --------------------------------------------------
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ double shfl_up_f64(double v, int d) {
  int lo = __double2loint(v), hi = __double2hiint(v);
  lo = __shfl_up_sync(0xFFFFFFFFu, lo, d);
  hi = __shfl_up_sync(0xFFFFFFFFu, hi, d);
  return __hiloint2double(hi, lo);
}
__device__ __forceinline__ double shfl_xor_f64(double v, int d) {
  int lo = __double2loint(v), hi = __double2hiint(v);
  lo = __shfl_xor_sync(0xFFFFFFFFu, lo, d);
  hi = __shfl_xor_sync(0xFFFFFFFFu, hi, d);
  return __hiloint2double(hi, lo);
}
__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, int d) {
  uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
  lo = __shfl_xor_sync(0xFFFFFFFFu, lo, d);
  hi = __shfl_xor_sync(0xFFFFFFFFu, hi, d);
  return ((uint64_t)hi << 32) | lo;
}

// Inclusive block scan (sum) over one value per thread.  `scratch` holds >= 33 T's.
// Returns the inclusive prefix; *total receives the block sum.  Fixed tree: deterministic.
template <typename T, typename ShflUp>
__device__ __forceinline__ T block_scan_incl(T v, T* scratch, T* total, ShflUp shfl_up) {
  const int lane = lane_id(), w = warp_id(), nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    T n = shfl_up(v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) scratch[w] = v;
  __syncthreads();
  if (w == 0) {
    T s = (lane < nw) ? scratch[lane] : T(0);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      T n = shfl_up(s, o);
      if (lane >= o) s += n;
    }
    scratch[lane] = s;
  }
  __syncthreads();
  T base = (w > 0) ? scratch[w - 1] : T(0);
  if (total) *total = scratch[nw - 1];
  __syncthreads();
  return v + base;
}
struct ShflUpI32 { __device__ int operator()(int v, int d) const { return __shfl_up_sync(0xFFFFFFFFu, v, d); } };
struct ShflUpU32 { __device__ uint32_t operator()(uint32_t v, int d) const { return __shfl_up_sync(0xFFFFFFFFu, v, d); } };
struct ShflUpF32 { __device__ float operator()(float v, int d) const { return __shfl_up_sync(0xFFFFFFFFu, v, d); } };
struct ShflUpF64 { __device__ double operator()(double v, int d) const { return shfl_up_f64(v, d); } };

// ---- in-shared-memory bitonic sort of `n` (power of two) u64 items, ascending -----
__device__ __forceinline__ void block_bitonic_sort_u64(uint64_t* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
        int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        int hi = lo | j;
        uint64_t x = a[lo], y = a[hi];
        bool up = ((lo & k) == 0);
        if ((x > y) == up) { a[lo] = y; a[hi] = x; }
      }
      __syncthreads();
    }
  }
}

// ---- threefry2x32, 20 rounds ---------------------------------------------------
__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }
__device__ __forceinline__ void threefry2x32(uint32_t k0, uint32_t k1, uint32_t& x0, uint32_t& x1) {
  const uint32_t k2 = k0 ^ k1 ^ 0x1BD11BDAu;
  x0 += k0; x1 += k1;
#define TLX_TF_ROUND(r) { x0 += x1; x1 = rotl32(x1, r); x1 ^= x0; }
  TLX_TF_ROUND(13) TLX_TF_ROUND(15) TLX_TF_ROUND(26) TLX_TF_ROUND(6)
  x0 += k1; x1 += k2 + 1u;
  TLX_TF_ROUND(17) TLX_TF_ROUND(29) TLX_TF_ROUND(16) TLX_TF_ROUND(24)
  x0 += k2; x1 += k0 + 2u;
  TLX_TF_ROUND(13) TLX_TF_ROUND(15) TLX_TF_ROUND(26) TLX_TF_ROUND(6)
  x0 += k0; x1 += k1 + 3u;
  TLX_TF_ROUND(17) TLX_TF_ROUND(29) TLX_TF_ROUND(16) TLX_TF_ROUND(24)
  x0 += k1; x1 += k2 + 4u;
  TLX_TF_ROUND(13) TLX_TF_ROUND(15) TLX_TF_ROUND(26) TLX_TF_ROUND(6)
  x0 += k2; x1 += k0 + 5u;
#undef TLX_TF_ROUND
}
// The sampler's uniform in [tiny, 1): bits -> [0,1) by the mantissa trick, then
// max(tiny, f * (1 - tiny) + tiny) which in f32 is f for f > 0 and tiny for f == 0.
__device__ __forceinline__ float threefry_uniform01(uint32_t k0, uint32_t k1, uint32_t counter_lo) {
  uint32_t x0 = 0u, x1 = counter_lo;
  threefry2x32(k0, k1, x0, x1);
  uint32_t bits = x0 ^ x1;
  return __uint_as_float((bits >> 9) | 0x3F800000u) - 1.0f;
}

// Out-of-line copy for the samplers, which read noise at many places: the twenty rounds inlined
// at each of them made their kernels outgrow the instruction cache.
static __device__ __noinline__ float threefry_uniform01_call(uint32_t k0, uint32_t k1, uint32_t counter_lo) {
  return threefry_uniform01(k0, k1, counter_lo);
}

// ---- Gumbel noise ---------------------------------------------------------------
// Exact form: evaluated in f64, rounded to f32 once (bit-identical to the CPU checker).
// Out of line on purpose (two f64 logarithms, used at many places, on few elements).
static __device__ __noinline__ float gumbel_exact(float u) {
  double d = (double)fmaxf(u, kF32Tiny);
  return (float)(-log(-log(d)));
}
// Screening form, f32; |gumbel_fast - gumbel_exact| is far below kGumbelSlack.
__device__ __forceinline__ float gumbel_fast(float u) {
  return -logf(-logf(fmaxf(u, kF32Tiny)));
}
// Cheapest screening form: hardware log2 for both logs.  -log(u) loses relative accuracy as u -> 1,
// so the last percent takes the series of -log(1 - d), d = 1 - u (exact in f32), to the fourth
// order (relative error below 1e-8); elsewhere the absolute error of the result stays below 5e-5.
// Branch-free: a rare slow branch would be paid by the whole warp.
__device__ __forceinline__ float gumbel_screen(float u) {
  u = fmaxf(u, kF32Tiny);
  const float d = 1.0f - u;
  const float series = d * fmaf(d, fmaf(d, fmaf(d, 0.25f, 0.33333334f), 0.5f), 1.0f);
  const float l = u > 0.99f ? series : -__logf(u);
  return -__logf(l);
}
constexpr float kGumbelSlack = 1e-3f;

// ---- checked build ------------------------------------------------------------------------------
// python -m tallax_b200.build --checked compiles with TLX_CHECKED: TLX_IN_BOUNDS(i, n, site) then tests an
// index that the code relies on being in range (it is false, and the access is skipped, when it is not) and
// records the first violation in a device word that tlx_debug_check_status reads.  In other builds the
// macro is the constant `true` and costs nothing.  It stands in for a memory checker where none can be
// run; the sites are the shared-memory and workspace indices of the streaming sampler.
#ifdef TLX_CHECKED
static __device__ int g_tlx_check_word[4];   // violations so far; site, index and bound of the first
__device__ __forceinline__ bool tlx_check_fail(int site, long long i, long long n) {
  if (atomicAdd(&g_tlx_check_word[0], 1) == 0) {
    g_tlx_check_word[1] = site;
    g_tlx_check_word[2] = (int)i;
    g_tlx_check_word[3] = (int)n;
  }
  return false;
}
#define TLX_IN_BOUNDS(i, n, site) \
  (((unsigned long long)(long long)(i) < (unsigned long long)(long long)(n)) || tlx_check_fail((site), (long long)(i), (long long)(n)))
#else
#define TLX_IN_BOUNDS(i, n, site) true
#endif

// Noise source shared by the samplers: dense tensor or threefry key.
// The key and the row offset may also be given as device operands (the *_dev entry points): the key as
// two words in device memory, the offset as an int32 scalar in device memory that is added to every row
// index.  A caller under a tracing compiler has both only as device buffers.
struct NoiseSrc {
  const float* dense;     // nullable
  int64_t stride;         // elements per row of `dense`
  uint32_t k0, k1;        // threefry key (unless key_dev)
  int64_t vocab;          // counter = row * vocab + token
  const uint32_t* key_dev;         // nullable: the key's two words in device memory
  const int32_t* row_offset_dev;   // nullable: added to the row index
  __device__ __forceinline__ int64_t row_of(int64_t row) const {
    return row_offset_dev ? row + (int64_t)__ldg(row_offset_dev) : row;
  }
  // start of the noise of a row (dense noise only)
  __device__ __forceinline__ const float* dense_row(int64_t row) const { return dense + row_of(row) * stride; }
  __device__ __forceinline__ float at(int64_t row, int64_t tok) const {
    row = row_of(row);
    if (dense) return __ldg(dense + row * stride + tok);
    const uint32_t a = key_dev ? __ldg(key_dev) : k0, b = key_dev ? __ldg(key_dev + 1) : k1;
    float f = threefry_uniform01_call(a, b, (uint32_t)(row * vocab + tok));
    return fmaxf(f, kF32Tiny);
  }
};

// (score, token) arg-max combine: larger score wins, equal scores -> lower token.
struct Best {
  float y;
  int tok;
};
__device__ __forceinline__ Best best_of(Best a, Best b) {
  bool take_b = (b.y > a.y) || (b.y == a.y && b.tok < a.tok);
  return take_b ? b : a;
}
__device__ __forceinline__ Best warp_best(Best v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best n;
    n.y = __shfl_xor_sync(0xFFFFFFFFu, v.y, o);
    n.tok = __shfl_xor_sync(0xFFFFFFFFu, v.tok, o);
    v = best_of(v, n);
  }
  return v;
}

}  // namespace tlx
