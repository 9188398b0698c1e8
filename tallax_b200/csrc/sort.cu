// Stable row-wise argsort: bitonic network on 64-bit composites (key << 32 | position).
//
// The position in the low word makes every composite unique, so the (unstable) bitonic
// network yields the stable order, and one u64 compare is the whole lexicographic test.
// Rows up to kTile elements are sorted entirely in shared memory by one CTA.  Longer
// rows keep the composites in the caller's workspace (L2-resident for the sizes of
// interest): tiles are sorted in shared memory, every merge stage then runs its far
// substages (partner distance >= kTile) over the workspace and its near substages in
// shared memory again.
// Substages are taken three at a time wherever possible: a thread brings eight elements
// (spaced by the smallest of the three distances) into registers, does the twelve
// compare-exchanges there and writes them back, which divides the shared-memory (or workspace)
// traffic and the barriers by three.
#include <mutex>

#include "tlx_common.cuh"

namespace tlx {

constexpr int kTile = 16384;    // composites per shared-memory tile (128 KB)
constexpr int kSortThreads = 1024;
constexpr uint64_t kPad = ~0ull;

template <int DT>
__device__ __forceinline__ uint64_t make_composite(const typename Elem<DT>::type* __restrict__ krow,
                                                   const int32_t* __restrict__ prow, int64_t c, int64_t n,
                                                   bool descending) {
  if (c >= n) return kPad;
  const int64_t src = prow ? (int64_t)prow[c] : c;
  uint32_t k = Elem<DT>::key(krow[src]);
  if (descending) k = ~k;
  return ((uint64_t)k << 32) | (uint32_t)c;
}

// Shared tiles are padded by one slot per eight: a thread that owns eight consecutive elements
// (the last substages of every stage) then strides 72 bytes instead of 64, which spreads a warp
// over all banks.
__device__ __forceinline__ int pad_idx(int i) { return i + (i >> 3); }
constexpr size_t padded_bytes(size_t elems) { return (elems + (elems >> 3)) * 8; }

__device__ __forceinline__ void cas_reg(uint64_t& x, uint64_t& y, bool up) {
  const bool swap = (x > y) == up;
  const uint64_t lo = swap ? y : x, hi = swap ? x : y;
  x = lo;
  y = hi;
}

// 2^NSUB elements e[b] = a[b * jl] (jl = the smallest of NSUB consecutive distances): the
// substages with distances jl << (NSUB-1), ..., jl in registers.
template <int NSUB>
__device__ __forceinline__ void butterfly(uint64_t (&e)[1 << NSUB], bool up) {
#pragma unroll
  for (int sub = NSUB - 1; sub >= 0; --sub) {
#pragma unroll
    for (int b = 0; b < (1 << NSUB); ++b)
      if (!(b & (1 << sub))) cas_reg(e[b], e[b | (1 << sub)], up);
  }
}

template <int NSUB>
__device__ __forceinline__ void tile_group(uint64_t* a, int tile, int64_t base, int64_t k, int jl) {
  constexpr int kSets = 1;   // element sets per thread and turn (two cost more in spills than they gain in overlap)
  const int items = tile >> NSUB;
  for (int t0 = threadIdx.x; t0 < items; t0 += kSets * (int)blockDim.x) {
    uint64_t e[kSets][1 << NSUB];
    int lo[kSets];
#pragma unroll
    for (int u = 0; u < kSets; ++u) {
      const int t = t0 + u * (int)blockDim.x;
      lo[u] = ((t & ~(jl - 1)) << NSUB) | (t & (jl - 1));
      if (t < items) {
#pragma unroll
        for (int b = 0; b < (1 << NSUB); ++b) e[u][b] = a[pad_idx(lo[u] + b * jl)];
      }
    }
#pragma unroll
    for (int u = 0; u < kSets; ++u)
      if (t0 + u * (int)blockDim.x < items) butterfly<NSUB>(e[u], ((base + lo[u]) & k) == 0);
#pragma unroll
    for (int u = 0; u < kSets; ++u) {
      if (t0 + u * (int)blockDim.x < items) {
#pragma unroll
        for (int b = 0; b < (1 << NSUB); ++b) a[pad_idx(lo[u] + b * jl)] = e[u][b];
      }
    }
  }
  __syncthreads();
}

// Substages j = j_from .. 1 of merge stage k on a shared tile whose first element has
// global index `base` in its row.
__device__ __forceinline__ void tile_substages(uint64_t* a, int tile, int64_t base, int64_t k, int j_from) {
  int j = j_from;
  for (; j >= 4; j >>= 3) tile_group<3>(a, tile, base, k, j >> 2);
  if (j == 2) tile_group<2>(a, tile, base, k, 1);
  else if (j == 1) tile_group<1>(a, tile, base, k, 1);
}

template <int DT>
__device__ __forceinline__ void emit(uint64_t v, int64_t c, int64_t n, bool descending,
                                     const int32_t* __restrict__ prow, typename Elem<DT>::type* __restrict__ okeys,
                                     int32_t* __restrict__ operm) {
  if (c >= n) return;
  uint32_t k = (uint32_t)(v >> 32);
  if (descending) k = ~k;
  const int32_t pos = (int32_t)(uint32_t)v;
  if (okeys) okeys[c] = Elem<DT>::from_key(k);
  if (operm) operm[c] = prow ? prow[pos] : pos;
}

// Whole row in one tile: build, sort, emit.  n_pad (power of two) <= kTile.
template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_small_kernel(
    const typename Elem<DT>::type* __restrict__ keys, const int32_t* __restrict__ in_perm, int64_t n, int n_pad,
    int descending, typename Elem<DT>::type* __restrict__ out_keys, int32_t* __restrict__ out_perm) {
  extern __shared__ uint64_t tile_smem[];
  const int64_t r = blockIdx.x;
  const auto* krow = keys + r * n;
  const int32_t* prow = in_perm ? in_perm + r * n : nullptr;
  for (int c = threadIdx.x; c < n_pad; c += blockDim.x)
    tile_smem[pad_idx(c)] = make_composite<DT>(krow, prow, c, n, descending);
  __syncthreads();
  for (int k = 2; k <= n_pad; k <<= 1) tile_substages(tile_smem, n_pad, 0, k, k >> 1);
  for (int c = threadIdx.x; c < n_pad; c += blockDim.x)
    emit<DT>(tile_smem[pad_idx(c)], c, n, descending, prow, out_keys ? out_keys + r * n : nullptr,
             out_perm ? out_perm + r * n : nullptr);
}

// Long rows, step 1: build composites of one tile and run stages 2..kTile on it.
template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_tiles_kernel(
    const typename Elem<DT>::type* __restrict__ keys, const int32_t* __restrict__ in_perm, int64_t n, int64_t n_pad,
    int descending, uint64_t* __restrict__ ws) {
  extern __shared__ uint64_t tile_smem[];
  const int64_t tiles_per_row = n_pad / kTile;
  const int64_t r = blockIdx.x / tiles_per_row;
  const int64_t base = (blockIdx.x % tiles_per_row) * kTile;
  const auto* krow = keys + r * n;
  const int32_t* prow = in_perm ? in_perm + r * n : nullptr;
  for (int c = threadIdx.x; c < kTile; c += blockDim.x)
    tile_smem[pad_idx(c)] = make_composite<DT>(krow, prow, base + c, n, descending);
  __syncthreads();
  for (int k = 2; k <= kTile; k <<= 1) tile_substages(tile_smem, kTile, base, k, k >> 1);
  uint64_t* dst = ws + r * n_pad + base;
  for (int c = threadIdx.x; c < kTile; c += blockDim.x) dst[c] = tile_smem[pad_idx(c)];
}

// Long rows, step 2: NSUB consecutive far substages (partner distances j1, j1/2, ... >= kTile) of stage k.
template <int NSUB>
__global__ void sort_far_kernel(uint64_t* __restrict__ ws, int64_t n_pad, int64_t rows, int64_t k, int64_t j1) {
  const int64_t per_row = n_pad >> NSUB;
  const int64_t total = rows * per_row;
  const int64_t jl = j1 >> (NSUB - 1);
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / per_row;
    const int64_t p = t - r * per_row;
    const int64_t lo = ((p & ~(jl - 1)) << NSUB) | (p & (jl - 1));
    uint64_t* a = ws + r * n_pad + lo;
    uint64_t e[1 << NSUB];
#pragma unroll
    for (int b = 0; b < (1 << NSUB); ++b) e[b] = a[b * jl];
    butterfly<NSUB>(e, (lo & k) == 0);
#pragma unroll
    for (int b = 0; b < (1 << NSUB); ++b) a[b * jl] = e[b];
  }
}

// Long rows, step 3: near substages (j < kTile) of stage k in shared memory; the last
// stage emits keys / permutation instead of writing the workspace back.
template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_near_kernel(
    uint64_t* __restrict__ ws, int64_t n, int64_t n_pad, int64_t k, int last, int descending,
    const int32_t* __restrict__ in_perm, typename Elem<DT>::type* __restrict__ out_keys,
    int32_t* __restrict__ out_perm) {
  extern __shared__ uint64_t tile_smem[];
  const int64_t tiles_per_row = n_pad / kTile;
  const int64_t r = blockIdx.x / tiles_per_row;
  const int64_t base = (blockIdx.x % tiles_per_row) * kTile;
  uint64_t* src = ws + r * n_pad + base;
  for (int c = threadIdx.x; c < kTile; c += blockDim.x) tile_smem[pad_idx(c)] = src[c];
  __syncthreads();
  tile_substages(tile_smem, kTile, base, k, kTile >> 1);
  if (!last) {
    for (int c = threadIdx.x; c < kTile; c += blockDim.x) src[c] = tile_smem[pad_idx(c)];
  } else {
    const int32_t* prow = in_perm ? in_perm + r * n : nullptr;
    for (int c = threadIdx.x; c < kTile; c += blockDim.x)
      emit<DT>(tile_smem[pad_idx(c)], base + c, n, descending, prow, out_keys ? out_keys + r * n : nullptr,
               out_perm ? out_perm + r * n : nullptr);
  }
}

// Raises a kernel's dynamic shared memory limit once per (kernel, device).
static int sort_smem(const void* func, size_t bytes) {
  if (bytes <= 48 * 1024) return TLX_OK;
  struct Entry { const void* func; int dev; size_t bytes; };
  static Entry cache[64];
  static int used = 0;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].func == func && cache[i].dev == dev && cache[i].bytes >= bytes) return TLX_OK;
  cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "sort: cudaFuncSetAttribute(%zu): %s", bytes, cudaGetErrorString(e));
  if (used < 64) cache[used++] = Entry{func, dev, bytes};
  return TLX_OK;
}

static int64_t next_pow2(int64_t n) {
  int64_t p = 1;
  while (p < n) p <<= 1;
  return p;
}

template <int DT>
static int sort_dispatch(cudaStream_t st, const void* keys, int64_t rows, int64_t n, int descending,
                         const int32_t* in_perm, void* out_keys, int32_t* out_perm, void* workspace,
                         size_t workspace_bytes) {
  using T = typename Elem<DT>::type;
  const int64_t n_pad = next_pow2(n < 2 ? 2 : n);
  int rc;
  if (n_pad <= kTile) {
    int threads = (int)(n_pad / 8);
    threads = threads < 64 ? 64 : (threads > kSortThreads ? kSortThreads : threads);
    if ((rc = sort_smem((const void*)sort_small_kernel<DT>, padded_bytes((size_t)n_pad))) != TLX_OK) return rc;
    sort_small_kernel<DT><<<(unsigned)rows, threads, padded_bytes((size_t)n_pad), st>>>(
        (const T*)keys, in_perm, n, (int)n_pad, descending, (T*)out_keys, out_perm);
    TLX_CHECK_LAUNCH("sort (single tile)");
    return TLX_OK;
  }
  const size_t need = (size_t)rows * (size_t)n_pad * 8;
  if (!workspace || workspace_bytes < need)
    return set_error(TLX_ERR_WORKSPACE, "sort: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  uint64_t* ws = (uint64_t*)workspace;
  const unsigned tiles = (unsigned)(rows * (n_pad / kTile));
  const size_t smem = padded_bytes((size_t)kTile);
  if ((rc = sort_smem((const void*)sort_tiles_kernel<DT>, smem)) != TLX_OK) return rc;
  if ((rc = sort_smem((const void*)sort_near_kernel<DT>, smem)) != TLX_OK) return rc;
  sort_tiles_kernel<DT><<<tiles, kSortThreads, smem, st>>>((const T*)keys, in_perm, n, n_pad, descending, ws);
  TLX_CHECK_LAUNCH("sort (tiles)");
  auto far_blocks = [&](int nsub) {
    const int64_t work = (rows * (n_pad >> nsub) + 255) / 256;
    return (unsigned)(work < 148 * 16 ? work : 148 * 16);
  };
  for (int64_t k = (int64_t)kTile * 2; k <= n_pad; k <<= 1) {
    int64_t j = k >> 1;
    while (j >= kTile) {   // the far substages, up to three per pass over the workspace
      int nsub = 0;
      for (int64_t jj = j; jj >= kTile && nsub < 3; jj >>= 1) ++nsub;
      if (nsub == 3) sort_far_kernel<3><<<far_blocks(3), 256, 0, st>>>(ws, n_pad, rows, k, j);
      else if (nsub == 2) sort_far_kernel<2><<<far_blocks(2), 256, 0, st>>>(ws, n_pad, rows, k, j);
      else sort_far_kernel<1><<<far_blocks(1), 256, 0, st>>>(ws, n_pad, rows, k, j);
      TLX_CHECK_LAUNCH("sort (far substages)");
      j >>= nsub;
    }
    sort_near_kernel<DT><<<tiles, kSortThreads, smem, st>>>(ws, n, n_pad, k, k == n_pad, descending, in_perm,
                                                             (T*)out_keys, out_perm);
    TLX_CHECK_LAUNCH("sort (near substages)");
  }
  return TLX_OK;
}

// Scratch of tlx_sort_static: lives in the library's image on every GPU that loads it.
constexpr size_t kStaticSortBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_sort_scratch[kStaticSortBytes];

}  // namespace tlx

using namespace tlx;

extern "C" {

size_t tlx_sort_workspace_bytes(int64_t rows, int64_t n) {
  if (rows <= 0 || n <= 0) return 0;
  const int64_t n_pad = next_pow2(n < 2 ? 2 : n);
  if (n_pad <= kTile) return 0;
  return (size_t)rows * (size_t)n_pad * 8;
}

int tlx_sort(void* stream, const void* keys, int dtype, int64_t rows, int64_t n, int descending,
             const int32_t* in_perm, void* out_keys, int32_t* out_perm, void* workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && n >= 0, "sort: negative extent");
  if (rows == 0 || n == 0) return TLX_OK;
  TLX_CHECK_ARG(keys, "sort: null keys");
  TLX_CHECK_ARG(out_keys || out_perm, "sort: no output requested");
  TLX_CHECK_ARG(n < (1ll << 31), "sort: row length %lld does not fit an int32 position", (long long)n);
  TLX_CHECK_ARG(rows * (next_pow2(n) / (n > kTile ? kTile : next_pow2(n))) < (1ll << 31), "sort: too many tiles");
  switch (dtype) {
    case TLX_F32: return sort_dispatch<TLX_F32>(st, keys, rows, n, descending, in_perm, out_keys, out_perm, workspace, workspace_bytes);
    case TLX_BF16: return sort_dispatch<TLX_BF16>(st, keys, rows, n, descending, in_perm, out_keys, out_perm, workspace, workspace_bytes);
    case TLX_F16: return sort_dispatch<TLX_F16>(st, keys, rows, n, descending, in_perm, out_keys, out_perm, workspace, workspace_bytes);
    case TLX_I32: return sort_dispatch<TLX_I32>(st, keys, rows, n, descending, in_perm, out_keys, out_perm, workspace, workspace_bytes);
    case TLX_U32: return sort_dispatch<TLX_U32>(st, keys, rows, n, descending, in_perm, out_keys, out_perm, workspace, workspace_bytes);
    default: return set_error(TLX_ERR_UNSUPPORTED, "sort: dtype %d not supported", dtype);
  }
}

size_t tlx_sort_static_max_bytes(void) { return kStaticSortBytes; }

int tlx_sort_static(void* stream, const void* keys, int dtype, int64_t rows, int64_t n, int descending,
                    const int32_t* in_perm, void* out_keys, int32_t* out_perm) {
  // The size check comes first and touches no CUDA state.
  const size_t need = tlx_sort_workspace_bytes(rows, n);
  if (need > kStaticSortBytes)
    return set_error(TLX_ERR_INVALID,
                     "sort_static: %lld rows of %lld keys need %zu bytes of scratch, the built-in area holds %zu; "
                     "use tlx_sort with a caller-provided workspace",
                     (long long)rows, (long long)n, need, (size_t)kStaticSortBytes);
  // In host code the array's name is only a handle: the device address is looked up once per
  // device (with that device current) and remembered.
  static void* device_address[64] = {};
  static std::mutex address_mutex;   // host threads may make their first calls at the same time
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "sort_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return set_error(TLX_ERR_UNSUPPORTED, "sort_static: device ordinal %d not supported", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(address_mutex);
    if (!device_address[dev]) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_sort_scratch);
      if (e != cudaSuccess || !ptr)
        return set_error(TLX_ERR_CUDA, "sort_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      device_address[dev] = ptr;
    }
    scratch = device_address[dev];
  }
  return tlx_sort(stream, keys, dtype, rows, n, descending, in_perm, out_keys, out_perm, scratch, kStaticSortBytes);
}

}  // extern "C"
