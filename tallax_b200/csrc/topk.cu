// Row-wise exact / single-pass top-k and the per-shard candidate stage of the
// vocab-sharded sampler.  One CTA per row: the streaming collector leaves a superset of
// the top-k in shared memory, a bitonic network orders it by (value desc, index asc).
#include "select.cuh"

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
};

template <int DT>
__device__ __forceinline__ typename Elem<DT>::type cast_replace(double v) {
  if constexpr (DT == TLX_F32) return (float)v;
  else if constexpr (DT == TLX_BF16) return __float2bfloat16_rn((float)v);
  else if constexpr (DT == TLX_F16) return __float2half_rn((float)v);
  else if constexpr (DT == TLX_I32) return (int32_t)v;
  else return (uint32_t)v;
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

  const int k_row = p.k_per_row ? p.k_per_row[r] : K;
  for (int j = threadIdx.x; j < K; j += blockDim.x) {
    const uint64_t c = cand[j];
    const int32_t col = (int32_t)cand_low(c);
    const bool have = j < m;
    if (p.cand_vals) {
      // candidate stage: f32 value, global token id, noise at that token
      const float v = have ? elem_as_float<DT>(row[col]) : -INFINITY;
      const int64_t tok = (int64_t)col + p.col_offset;
      p.cand_vals[r * K + j] = v;
      p.cand_idx[r * K + j] = have ? (int32_t)tok : -1;
      float u = 0.5f;
      if (have) u = p.noise.dense ? __ldg(p.noise.dense + r * p.noise.stride + col) : p.noise.at(r + p.dim0_offset, tok);
      p.cand_noise[r * K + j] = u;
    } else {
      T v = have ? row[col] : cast_replace<DT>(0.0);
      if (p.use_replace && j >= k_row) v = cast_replace<DT>(p.replace_val);
      reinterpret_cast<T*>(p.out_vals)[r * K + j] = v;
      p.out_idx[r * K + j] = have ? col : 0;
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
                                 float* out_vals, int32_t* out_idx, float* out_noise) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && v_local > 0, "shard_candidates: bad extent");
  TLX_CHECK_ARG(k_cand >= 1 && k_cand <= 1024, "shard_candidates: k_cand must be in [1, 1024], got %d", k_cand);
  TLX_CHECK_ARG((int64_t)k_cand <= v_local, "shard_candidates: k_cand exceeds the shard width");
  TLX_CHECK_ARG(dtype == TLX_F32 || dtype == TLX_BF16 || dtype == TLX_F16, "shard_candidates: float logits only");
  TLX_CHECK_ARG(row_stride >= v_local, "shard_candidates: row stride smaller than the row");
  TLX_CHECK_ARG(col_offset >= 0 && col_offset + v_local <= (1ll << 31), "shard_candidates: token ids exceed int32");
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(logits && out_vals && out_idx && out_noise, "shard_candidates: null pointer");
  TopkParams p{};
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

}  // extern "C"
