// Stable row-wise argsort: bitonic network on 64-bit composites (key << 32 | position).
//
// The position in the low word makes every composite unique, so the (unstable) bitonic
// network yields the stable order, and one u64 compare is the whole lexicographic test.
// Rows up to kTile elements are sorted entirely in shared memory by one CTA.  Longer
// rows keep the composites in the caller's workspace (L2-resident for the sizes of
// interest): tiles are sorted in shared memory, every merge stage then runs its far
// substages (partner distance >= kTile) over the workspace and its near substages in
// shared memory again.
#include "tlx_common.cuh"

namespace tlx {

constexpr int kTile = 4096;     // composites per shared-memory tile (32 KB)
constexpr int kSortThreads = 512;
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

__device__ __forceinline__ void cas(uint64_t* a, int lo, int hi, bool up) {
  uint64_t x = a[lo], y = a[hi];
  if ((x > y) == up) { a[lo] = y; a[hi] = x; }
}

// Substages j = j_from .. 1 of merge stage k on a shared tile whose first element has
// global index `base` in its row.
__device__ __forceinline__ void tile_substages(uint64_t* a, int tile, int64_t base, int64_t k, int j_from) {
  for (int j = j_from; j > 0; j >>= 1) {
    for (int t = threadIdx.x; t < (tile >> 1); t += blockDim.x) {
      const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
      cas(a, lo, lo | j, ((base + lo) & k) == 0);
    }
    __syncthreads();
  }
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
  for (int c = threadIdx.x; c < n_pad; c += blockDim.x) tile_smem[c] = make_composite<DT>(krow, prow, c, n, descending);
  __syncthreads();
  for (int k = 2; k <= n_pad; k <<= 1) tile_substages(tile_smem, n_pad, 0, k, k >> 1);
  for (int c = threadIdx.x; c < n_pad; c += blockDim.x)
    emit<DT>(tile_smem[c], c, n, descending, prow, out_keys ? out_keys + r * n : nullptr,
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
    tile_smem[c] = make_composite<DT>(krow, prow, base + c, n, descending);
  __syncthreads();
  for (int k = 2; k <= kTile; k <<= 1) tile_substages(tile_smem, kTile, base, k, k >> 1);
  uint64_t* dst = ws + r * n_pad + base;
  for (int c = threadIdx.x; c < kTile; c += blockDim.x) dst[c] = tile_smem[c];
}

// Long rows, step 2: one far substage (partner distance j >= kTile) of stage k.
__global__ void sort_far_substage_kernel(uint64_t* __restrict__ ws, int64_t n_pad, int64_t rows, int64_t k, int64_t j) {
  const int64_t half = n_pad >> 1;
  const int64_t total = rows * half;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / half;
    const int64_t p = t - r * half;
    const int64_t lo = ((p & ~(j - 1)) << 1) | (p & (j - 1));
    uint64_t* a = ws + r * n_pad;
    const uint64_t x = a[lo], y = a[lo | j];
    const bool up = (lo & k) == 0;
    if ((x > y) == up) { a[lo] = y; a[lo | j] = x; }
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
  for (int c = threadIdx.x; c < kTile; c += blockDim.x) tile_smem[c] = src[c];
  __syncthreads();
  tile_substages(tile_smem, kTile, base, k, kTile >> 1);
  if (!last) {
    for (int c = threadIdx.x; c < kTile; c += blockDim.x) src[c] = tile_smem[c];
  } else {
    const int32_t* prow = in_perm ? in_perm + r * n : nullptr;
    for (int c = threadIdx.x; c < kTile; c += blockDim.x)
      emit<DT>(tile_smem[c], base + c, n, descending, prow, out_keys ? out_keys + r * n : nullptr,
               out_perm ? out_perm + r * n : nullptr);
  }
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
  if (n_pad <= kTile) {
    sort_small_kernel<DT><<<(unsigned)rows, kSortThreads, (size_t)n_pad * 8, st>>>(
        (const T*)keys, in_perm, n, (int)n_pad, descending, (T*)out_keys, out_perm);
    TLX_CHECK_LAUNCH("sort (single tile)");
    return TLX_OK;
  }
  const size_t need = (size_t)rows * (size_t)n_pad * 8;
  if (!workspace || workspace_bytes < need)
    return set_error(TLX_ERR_WORKSPACE, "sort: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  uint64_t* ws = (uint64_t*)workspace;
  const unsigned tiles = (unsigned)(rows * (n_pad / kTile));
  const size_t smem = (size_t)kTile * 8;
  sort_tiles_kernel<DT><<<tiles, kSortThreads, smem, st>>>((const T*)keys, in_perm, n, n_pad, descending, ws);
  TLX_CHECK_LAUNCH("sort (tiles)");
  const int64_t pairs = rows * (n_pad >> 1);
  const unsigned far_blocks = (unsigned)((pairs + 255) / 256 < 148 * 16 ? (pairs + 255) / 256 : 148 * 16);
  for (int64_t k = (int64_t)kTile * 2; k <= n_pad; k <<= 1) {
    for (int64_t j = k >> 1; j >= kTile; j >>= 1) {
      sort_far_substage_kernel<<<far_blocks, 256, 0, st>>>(ws, n_pad, rows, k, j);
      TLX_CHECK_LAUNCH("sort (far substage)");
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
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "sort_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return set_error(TLX_ERR_UNSUPPORTED, "sort_static: device ordinal %d not supported", dev);
  if (!device_address[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_sort_scratch);
    if (e != cudaSuccess || !ptr)
      return set_error(TLX_ERR_CUDA, "sort_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    device_address[dev] = ptr;
  }
  return tlx_sort(stream, keys, dtype, rows, n, descending, in_perm, out_keys, out_perm, device_address[dev],
                  kStaticSortBytes);
}

}  // extern "C"
