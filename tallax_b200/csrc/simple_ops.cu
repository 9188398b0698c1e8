// Gather (take_along_axis), cumsum, arg-max and counter-based uniform noise.
// All four are plain HBM-bound streaming kernels: one read, one write, coalesced.
#include "tlx_common.cuh"

#include <atomic>

namespace tlx {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---------------------------------------------------------------------------------
// gather
// ---------------------------------------------------------------------------------
// Eight consecutive outputs per thread: two 16-byte index loads, eight independent random reads in flight,
// 16-byte stores.  The random reads are what the kernel waits for (a 32-byte DRAM sector per element), so
// the number a thread keeps in flight is what sets the rate.
template <typename T>
__global__ void __launch_bounds__(256) gather_axis1_kernel(const T* __restrict__ values, const int32_t* __restrict__ idx,
                                                           T* __restrict__ out, int64_t rows, int64_t vcols, int64_t icols) {
  constexpr int kPer = 8;
  const int64_t groups_per_row = (icols + kPer - 1) / kPer;
  const int64_t total = rows * groups_per_row;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / groups_per_row;
    const int64_t c0 = (g - r * groups_per_row) * kPer;
    const int32_t* ip = idx + r * icols + c0;
    const T* vrow = values + r * vcols;
    T* op = out + r * icols + c0;
    int32_t ii[kPer];
    const int n = (int)min((int64_t)kPer, icols - c0);
    if (n == kPer && ((reinterpret_cast<uintptr_t>(ip) & 15) == 0)) {
      const int4 a = __ldcs(reinterpret_cast<const int4*>(ip));
      const int4 b = __ldcs(reinterpret_cast<const int4*>(ip) + 1);
      ii[0] = a.x; ii[1] = a.y; ii[2] = a.z; ii[3] = a.w;
      ii[4] = b.x; ii[5] = b.y; ii[6] = b.z; ii[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < kPer; ++j) ii[j] = (j < n) ? __ldg(ip + j) : -1;
    }
    T o[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const bool ok = (j < n) && ii[j] >= 0 && (int64_t)ii[j] < vcols;
      o[j] = ok ? __ldg(vrow + ii[j]) : T(0);
    }
    if (n == kPer && sizeof(T) == 4 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
      uint4 w0, w1;
      memcpy(&w0, &o[0], 16);
      memcpy(&w1, &o[4], 16);
      __stcs(reinterpret_cast<uint4*>(op), w0);
      __stcs(reinterpret_cast<uint4*>(op) + 1, w1);
    } else {
#pragma unroll
      for (int j = 0; j < kPer; ++j) if (j < n) op[j] = o[j];
    }
  }
}

template <typename T>
__global__ void gather_axis0_kernel(const T* __restrict__ values, const int32_t* __restrict__ idx,
                                    T* __restrict__ out, int64_t vrows, int64_t cols, int64_t irows) {
  const int64_t total = irows * cols;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = e % cols;
    const int32_t i = __ldg(idx + e);
    const bool ok = i >= 0 && (int64_t)i < vrows;
    out[e] = ok ? __ldg(values + (int64_t)i * cols + c) : T(0);
  }
}

template <typename T>
static int launch_gather(cudaStream_t st, const void* values, const int32_t* idx, void* out, int64_t vr,
                         int64_t vc, int64_t ir, int64_t ic, int axis) {
  const int threads = 256;
  if (axis == 1) {
    const int64_t total = ir * ((ic + 7) >> 3);
    if (total == 0) return TLX_OK;
    const int64_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 64 ? want : 148 * 64);
    gather_axis1_kernel<T><<<blocks, threads, 0, st>>>((const T*)values, idx, (T*)out, ir, vc, ic);
  } else {
    const int64_t total = ir * ic;
    if (total == 0) return TLX_OK;
    const int64_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    gather_axis0_kernel<T><<<blocks, threads, 0, st>>>((const T*)values, idx, (T*)out, vr, vc, ir);
  }
  TLX_CHECK_LAUNCH("take_along_axis");
  return TLX_OK;
}

// ---------------------------------------------------------------------------------
// cumsum
// ---------------------------------------------------------------------------------
template <typename T, typename Shfl>
__global__ void cumsum_axis1_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t cols, int reverse) {
  constexpr int ITEMS = 4;
  __shared__ T scratch[33];
  const T* src = in + blockIdx.x * cols;
  T* dst = out + blockIdx.x * cols;
  T carry = T(0);
  const int64_t chunk = (int64_t)blockDim.x * ITEMS;
  for (int64_t base = 0; base < cols; base += chunk) {
    T v[ITEMS];
    T run = T(0);
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      const int64_t c = base + (int64_t)threadIdx.x * ITEMS + j;
      const int64_t cc = reverse ? (cols - 1 - c) : c;
      T x = (c < cols) ? src[cc] : T(0);
      run += x;
      v[j] = run;
    }
    T total;
    T incl = block_scan_incl<T>(run, scratch, &total, Shfl());
    const T offs = carry + (incl - run);
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      const int64_t c = base + (int64_t)threadIdx.x * ITEMS + j;
      const int64_t cc = reverse ? (cols - 1 - c) : c;
      if (c < cols) dst[cc] = v[j] + offs;
    }
    carry += total;
  }
}

template <typename T>
__global__ void cumsum_axis0_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols,
                                    int reverse) {
  const int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  T acc = T(0);
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t rr = reverse ? (rows - 1 - r) : r;
    acc += in[rr * cols + c];
    out[rr * cols + c] = acc;
  }
}

// ---------------------------------------------------------------------------------
// arg-max, lowest index on ties
// ---------------------------------------------------------------------------------
template <int DT>
__global__ void argmax_axis1_kernel(const typename Elem<DT>::type* __restrict__ x, int64_t cols,
                                    int32_t* __restrict__ out) {
  __shared__ uint64_t sbest[32];
  const typename Elem<DT>::type* row = x + blockIdx.x * cols;
  // composite: key in the high word, inverted column in the low word -> one u64 max
  uint64_t best = 0;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    uint64_t v = ((uint64_t)Elem<DT>::key(row[c]) << 32) | (uint32_t)(0x7FFFFFFF - (int32_t)c);
    best = v > best ? v : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    uint64_t n = shfl_xor_u64(best, o);
    best = n > best ? n : best;
  }
  if (lane_id() == 0) sbest[warp_id()] = best;
  __syncthreads();
  if (warp_id() == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane_id() < nw ? sbest[lane_id()] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      uint64_t n = shfl_xor_u64(best, o);
      best = n > best ? n : best;
    }
    if (lane_id() == 0) out[blockIdx.x] = 0x7FFFFFFF - (int32_t)(uint32_t)best;
  }
}

template <int DT>
__global__ void argmax_axis0_kernel(const typename Elem<DT>::type* __restrict__ x, int64_t rows, int64_t cols,
                                    int32_t* __restrict__ out) {
  const int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (c >= cols) return;
  uint32_t bk = 0;
  int32_t bi = 0;
  for (int64_t r = 0; r < rows; ++r) {
    uint32_t k = Elem<DT>::key(x[r * cols + c]);
    if (r == 0 || k > bk) { bk = k; bi = (int32_t)r; }
  }
  out[c] = bi;
}

template <int DT>
static int launch_argmax(cudaStream_t st, const void* keys, int64_t rows, int64_t cols, int axis, int32_t* out) {
  using T = typename Elem<DT>::type;
  if (axis == 1) {
    argmax_axis1_kernel<DT><<<(unsigned)rows, 256, 0, st>>>((const T*)keys, cols, out);
  } else {
    argmax_axis0_kernel<DT><<<(unsigned)((cols + 127) / 128), 128, 0, st>>>((const T*)keys, rows, cols, out);
  }
  TLX_CHECK_LAUNCH("argmax");
  return TLX_OK;
}

// ---------------------------------------------------------------------------------
// counter-based uniform noise at arbitrary (i0, i1)
// ---------------------------------------------------------------------------------
__global__ void sparse_uniform_kernel(uint32_t k0, uint32_t k1, const uint32_t* __restrict__ key_dev,
                                      const int32_t* __restrict__ i0, const int32_t* __restrict__ i1, int64_t count,
                                      int64_t dim1, float minval, float maxval, float* __restrict__ out) {
  if (key_dev) { k0 = __ldg(key_dev); k1 = __ldg(key_dev + 1); }   // the key as a device operand
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < count;
       e += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t ctr = (uint32_t)((int64_t)i0[e] * dim1 + (int64_t)i1[e]);
    const float f = threefry_uniform01(k0, k1, ctr);
    // separate multiply and add, as the reference computes them
    out[e] = fmaxf(minval, __fadd_rn(__fmul_rn(f, __fsub_rn(maxval, minval)), minval));
  }
}

// ---------------------------------------------------------------------------------
// key outputs in canonical form: what a float looks like after the round trip through the
// order-preserving key (-0 -> +0, every NaN -> the one canonical NaN), in place
// ---------------------------------------------------------------------------------
template <int DT>
__global__ void canonicalize_kernel(typename Elem<DT>::type* __restrict__ x, int64_t count) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < count; e += (int64_t)gridDim.x * blockDim.x)
    x[e] = Elem<DT>::from_key(Elem<DT>::key(x[e]));
}

}  // namespace tlx

using namespace tlx;

extern "C" {

int tlx_abi_version(void) { return TLX_ABI_VERSION; }
const char* tlx_last_error(void) { return tlx::g_err; }
unsigned long long tlx_kernel_launches(void) { return tlx::g_launches.load(std::memory_order_relaxed); }

int tlx_take_along_axis(void* stream, const void* values, const int32_t* indices, void* out, int64_t val_rows,
                        int64_t val_cols, int64_t idx_rows, int64_t idx_cols, int elem_bytes, int axis) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(axis == 0 || axis == 1, "take_along_axis: axis must be 0 or 1, got %d", axis);
  TLX_CHECK_ARG(val_rows >= 0 && val_cols >= 0 && idx_rows >= 0 && idx_cols >= 0, "take_along_axis: negative extent");
  if (axis == 1)
    TLX_CHECK_ARG(val_rows == idx_rows, "take_along_axis: batch extents differ (%lld vs %lld)", (long long)val_rows,
                  (long long)idx_rows);
  else
    TLX_CHECK_ARG(val_cols == idx_cols, "take_along_axis: batch extents differ (%lld vs %lld)", (long long)val_cols,
                  (long long)idx_cols);
  if (idx_rows * idx_cols == 0) return TLX_OK;
  TLX_CHECK_ARG(values && indices && out, "take_along_axis: null pointer");
  switch (elem_bytes) {
    case 1: return launch_gather<uint8_t>(st, values, indices, out, val_rows, val_cols, idx_rows, idx_cols, axis);
    case 2: return launch_gather<uint16_t>(st, values, indices, out, val_rows, val_cols, idx_rows, idx_cols, axis);
    case 4: return launch_gather<uint32_t>(st, values, indices, out, val_rows, val_cols, idx_rows, idx_cols, axis);
    case 8: return launch_gather<uint64_t>(st, values, indices, out, val_rows, val_cols, idx_rows, idx_cols, axis);
    default: return set_error(TLX_ERR_UNSUPPORTED, "take_along_axis: element size %d not supported", elem_bytes);
  }
}

int tlx_cumsum(void* stream, const void* in, void* out, int64_t rows, int64_t cols, int dtype, int axis,
               int reverse) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(axis == 0 || axis == 1, "cumsum: axis must be 0 or 1, got %d", axis);
  TLX_CHECK_ARG(rows >= 0 && cols >= 0, "cumsum: negative extent");
  if (rows * cols == 0) return TLX_OK;
  TLX_CHECK_ARG(in && out, "cumsum: null pointer");
  if (dtype != TLX_F32 && dtype != TLX_I32)
    return set_error(TLX_ERR_UNSUPPORTED, "cumsum: dtype %d not supported (f32, i32)", dtype);
  if (axis == 1) {
    if (dtype == TLX_F32)
      cumsum_axis1_kernel<float, ShflUpF32><<<(unsigned)rows, 256, 0, st>>>((const float*)in, (float*)out, cols, reverse);
    else
      cumsum_axis1_kernel<int, ShflUpI32><<<(unsigned)rows, 256, 0, st>>>((const int*)in, (int*)out, cols, reverse);
  } else {
    const unsigned blocks = (unsigned)((cols + 127) / 128);
    if (dtype == TLX_F32)
      cumsum_axis0_kernel<float><<<blocks, 128, 0, st>>>((const float*)in, (float*)out, rows, cols, reverse);
    else
      cumsum_axis0_kernel<int><<<blocks, 128, 0, st>>>((const int*)in, (int*)out, rows, cols, reverse);
  }
  TLX_CHECK_LAUNCH("cumsum");
  return TLX_OK;
}

int tlx_argmax(void* stream, const void* keys, int dtype, int64_t rows, int64_t cols, int axis, int32_t* out_idx) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(axis == 0 || axis == 1, "argmax: axis must be 0 or 1, got %d", axis);
  TLX_CHECK_ARG(rows > 0 && cols > 0, "argmax: empty input");
  TLX_CHECK_ARG(keys && out_idx, "argmax: null pointer");
  TLX_CHECK_ARG(rows < (1ll << 31) && cols < (1ll << 31), "argmax: extent too large");
  switch (dtype) {
    case TLX_F32: return launch_argmax<TLX_F32>(st, keys, rows, cols, axis, out_idx);
    case TLX_BF16: return launch_argmax<TLX_BF16>(st, keys, rows, cols, axis, out_idx);
    case TLX_F16: return launch_argmax<TLX_F16>(st, keys, rows, cols, axis, out_idx);
    case TLX_I32: return launch_argmax<TLX_I32>(st, keys, rows, cols, axis, out_idx);
    case TLX_U32: return launch_argmax<TLX_U32>(st, keys, rows, cols, axis, out_idx);
    default: return set_error(TLX_ERR_UNSUPPORTED, "argmax: dtype %d not supported", dtype);
  }
}

static int sparse_random_uniform_impl(void* stream, uint32_t key0, uint32_t key1, const uint32_t* key_dev,
                                      const int32_t* idx0, const int32_t* idx1, int64_t count, int64_t dim1_size,
                                      float minval, float maxval, float* out) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(count >= 0 && dim1_size > 0, "sparse_random_uniform: bad extent");
  if (count == 0) return TLX_OK;
  TLX_CHECK_ARG(idx0 && idx1 && out, "sparse_random_uniform: null pointer");
  const int64_t want = (count + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  sparse_uniform_kernel<<<blocks, 256, 0, st>>>(key0, key1, key_dev, idx0, idx1, count, dim1_size, minval, maxval, out);
  TLX_CHECK_LAUNCH("sparse_random_uniform");
  return TLX_OK;
}

int tlx_canonicalize_keys(void* stream, void* x, int dtype, int64_t count) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(count >= 0, "canonicalize_keys: negative extent");
  if (count == 0 || dtype == TLX_I32 || dtype == TLX_U32) return TLX_OK;   // integers are their own canonical form
  TLX_CHECK_ARG(x, "canonicalize_keys: null pointer");
  const int64_t want = (count + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  switch (dtype) {
    case TLX_F32: canonicalize_kernel<TLX_F32><<<blocks, 256, 0, st>>>((float*)x, count); break;
    case TLX_BF16: canonicalize_kernel<TLX_BF16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)x, count); break;
    case TLX_F16: canonicalize_kernel<TLX_F16><<<blocks, 256, 0, st>>>((__half*)x, count); break;
    default: return set_error(TLX_ERR_UNSUPPORTED, "canonicalize_keys: dtype %d not supported", dtype);
  }
  TLX_CHECK_LAUNCH("canonicalize_keys");
  return TLX_OK;
}

int tlx_sparse_random_uniform(void* stream, uint32_t key0, uint32_t key1, const int32_t* idx0, const int32_t* idx1,
                              int64_t count, int64_t dim1_size, float minval, float maxval, float* out) {
  return sparse_random_uniform_impl(stream, key0, key1, nullptr, idx0, idx1, count, dim1_size, minval, maxval, out);
}

int tlx_sparse_random_uniform_dev(void* stream, const uint32_t* key_dev, const int32_t* idx0, const int32_t* idx1,
                                  int64_t count, int64_t dim1_size, float minval, float maxval, float* out) {
  if (!key_dev) return set_error(TLX_ERR_INVALID, "sparse_random_uniform: null key");
  return sparse_random_uniform_impl(stream, 0u, 0u, key_dev, idx0, idx1, count, dim1_size, minval, maxval, out);
}

}  // extern "C"
