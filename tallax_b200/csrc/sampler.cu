// Fused temperature / top-k / top-p / noise sampler on [rows, vocab] logits, the
// candidate-level sampler, and the merge stage of the vocab-sharded sampler.
//
// Every row is seen as S interleaved slices (slice s = the 4 KB chunks s, s + S, ... of the row),
// each at most 28 KB, so that a slice is a sample of the whole row.  Slices are brought into
// shared memory with bulk copies (TMA, cp.async.bulk + mbarrier), two buffers per CTA: one is
// worked on while the next one arrives.  Logits are read from HBM once.
//
// tlx_sample, batches with at least one row per two CTA slots (the decode case):
//   rows kernel    one CTA per row.  Greedy rows keep a running arg-max.  Rows with
//                  1 <= top_k <= kFastK estimate a threshold bin on their first slice and note, per
//                  warp, the vectors that hold something at or above it (one packed compare per
//                  vector, one warp vote per four vectors a lane); the noted vectors are looked at
//                  densely once per slice and their passing elements appended to a candidate list
//                  in shared memory (the bin is raised exactly, from a histogram of the list, when
//                  the list fills up).  The row finishes inside the CTA: top-k boundary, softmax
//                  mass and top-p threshold from a histogram over the candidates' keys (bf16;
//                  sorted candidates for f32), Gumbel arg-max over the kept ones.
//                  Rows without any filter (top-k disabled and top_p >= 1) are streamed with their
//                  noise: Gumbel arg-max over the whole row.
//   cluster kernel (sampler_wide.cuh, bf16 rows whose top-k is disabled, top_p < 1) one cluster of eight CTAs
//                  per row keeps the row resident in shared memory; it runs on a side stream
//                  next to the rows kernel, since the two work on disjoint rows.
//   When the cluster kernel does not apply (rows not 16-byte aligned, vocabulary too long for the
//   cluster's shared memory) those rows take three steps instead:
//     slices kernel   (before the rows kernel) per slice: maximum, histogram of the 2048 16-bit
//                     keys below it, sum of exp(x - max) of everything lower;
//     rows kernel     adds the slices' histograms up, takes the top-p threshold from them (the
//                     mass of a value group is count * exp(value - max)) and stores it;
//     slices kernel   (final pass) per slice: Gumbel scores of the elements at or above the
//                     threshold, the slice's winner goes to the row with an atomic max, the CTA
//                     that delivers the last slice writes the token.
//   Rows with a top-k above kFastK, and f32 rows without top-k, are rare enough to take the
//   multi-pass whole-row routines of sampler_general.cuh.
// Small batches: all rows are cut into slices (slices kernel, candidates per slice and warp)
// and merged per row by the merge kernel, so that every SM streams whatever the batch size.
//
// Nothing on a per-slice path waits for a global-memory round trip (while the bulk copies
// saturate the memory system such a round trip costs microseconds).  Results are exact: a
// threshold estimate that turns out too high is detected (fewer than top_k candidates) and the
// row is streamed again with a lower one; the exact multi-pass select is the last resort.
// Routines that run once per row or less are kept out of line, which keeps the per-slice loops
// small in the instruction cache.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "sampler_general.cuh"
#include "exchange.cuh"

namespace tlx {

constexpr int kThreads = 256;        // slices kernel
constexpr int kRowThreads = 512;     // merge kernel
constexpr int kSliceBytes = 28672;   // one slice buffer (two per CTA)
constexpr int kChunkBytes = 4096;    // interleaving granule
constexpr int kChunksPerSlice = kSliceBytes / kChunkBytes;
constexpr int kRecordCap = 2048;     // candidates (u64) a slice may publish == 16 KB payload
constexpr int kMergeCap = 4096;      // candidates (u64) held in shared memory
constexpr int kWin = 2048;           // bf16 histogram window: 16 binades of 16-bit keys below the maximum
constexpr int kFastK = 2048;         // largest top_k served by the candidate path
constexpr int kSample = 2048;        // elements of a slice sampled for the first threshold
constexpr int kMaxSlices = 256;
constexpr uint32_t kWaitLimit = 1u << 24;  // bounded mbarrier polling

enum RowClass : int { kGreedy = 0, kFast = 1, kGeneral = 2 };
enum StatusBits : int { kStatusGeneral = 1, kStatusTimeout = 2, kStatusRedone = 4 };

constexpr int kWarps = kThreads / 32;
constexpr int kMaxWarps = 16;        // warps of the largest CTA that uses the per-warp result slots
constexpr int kRowsKThreads = 256;   // rows kernel
constexpr int kRowWarps = kRowsKThreads / 32;
constexpr int kWarpCap = kRecordCap / kWarps;   // candidates one warp may publish per slice
constexpr int kWarpHits = kSliceBytes / 16 / kWarps;   // vectors one warp owns in a slice
static_assert(kWarps <= 16, "SliceHeader holds 16 per-warp counts");
static_assert(kSliceBytes / 16 == kWarpHits * kWarps, "slice vectors must divide evenly among the warps");

struct SliceHeader {   // 64 bytes, one per (row, slice) in the workspace
  int cutoff_bin;      // candidates: every slice element with bin >= cutoff_bin was published
  int overflow;        // candidates: a warp's segment overflowed, the set is incomplete
  int kmax16;          // general/bf16: maximum 16-bit key of the slice
  float smax;          // general/bf16: slice maximum as a float
  unsigned long long top;  // greedy: arg-max composite (key << 32 | 0x7FFFFFFF - token)
  double mass;         // general/bf16: sum of exp(x - slice max)
  unsigned short wcount[16];  // candidates: entries in each warp's segment of the payload
};
static_assert(sizeof(SliceHeader) == 64, "SliceHeader layout");

// What the warps of a CTA leave behind for the thread that publishes the slice.
struct WarpResults {
  unsigned long long top[kMaxWarps];
  unsigned short count[kMaxWarps];
  unsigned short bin[kMaxWarps];
  unsigned char overflow[kMaxWarps];
  int cutoff_bin;
};

constexpr size_t kRecordBytes = sizeof(SliceHeader) + (size_t)kRecordCap * 8;

constexpr size_t kSharedHeader = (sizeof(SelectShared) + 15) & ~size_t(15);
constexpr size_t kUnionBytes = 32768;  // kMergeCap candidates (u64) == kHistBins f64 mass bins

// Per row, in the workspace: what the final pass over a row without top-k needs and leaves.
struct RowState {
  unsigned int min_key;        // elements with key >= min_key are kept ...
  float thr;                   // ... and satisfy !(x < thr)
  unsigned long long best;     // max over slices of key(score) << 32 | (0x7FFFFFFF - token)
  int done;                    // slices that have delivered their best
  int pad[3];
};
static_assert(sizeof(RowState) == 32, "RowState layout");

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
  // geometry
  int S;               // slices per row
  int chunk_elems;     // elements per chunk
  int nchunks;         // chunks per row (the last one may be partial)
  int use_tma;         // row starts and strides are 16-byte aligned
  int only_general;    // slices kernel: skip rows that the rows kernel finishes on its own
  int have_records;    // rows kernel: the slices kernel has written the records of the general rows
  int final_pass;      // slices kernel: score the kept elements of the general rows (third kernel)
  int wide_elsewhere;  // rows kernel: the rows without top-k are sampled by the cluster kernel
  RowState* rowstate;
  unsigned long long div_magic;  // ceil(2^40 / S)
  // workspace
  int32_t* counters;   // [1] set if a bounded wait gave up
  unsigned char* records;
  long long* timeline; // timeline builds only: 16 global-timer stamps per CTA (see TLX_STAMP)
};

// Timeline builds (python -m tallax_b200.build --timeline, a library of its own) record the global timer
// at marked points of the streaming path's kernels, 16 slots per CTA; other builds compile the marks away.
#ifdef TLX_TIMELINE
__device__ __forceinline__ long long global_timer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define TLX_STAMP(sp, k)                                                                              \
  do {                                                                                                \
    if (threadIdx.x == 0 && (sp).timeline) (sp).timeline[(size_t)blockIdx.x * 16 + (k)] = global_timer_ns(); \
  } while (0)
#else
#define TLX_STAMP(sp, k) do {} while (0)
#endif

struct __align__(16) Control {   // per-CTA bookkeeping in shared memory
  unsigned long long mbar[2];
  int item[2];
  int merge_flag[2];
  int timeout;
  int pad;
  WarpResults wr[2];
  int list_n;                 // slices kernel: this CTA's current batch of items
  int list[64];
  uint32_t list_cls[64];
  unsigned short rows_list[1024];   // slices kernel: the rows it works on, compacted
};

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false if the barrier did not complete within kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                          unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Release / acquire fence at GPU scope: orders this thread's (and, through a preceding barrier,
// its CTA's) writes before a following atomic, without the total order __threadfence() asks for.
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- slice geometry ---------------------------------------------------------------------
// Slice `sl` of a row owns the chunks sl, sl + S, sl + 2S, ...; they sit back to back in the
// slice buffer.  Only the row's last chunk can be partial, and it is then the last chunk
// of its slice.
struct Geometry {
  int S, chunk_elems, nchunks;
  int64_t n;
  int chunk_shift;  // chunk_elems is a power of two
  unsigned long long div_magic;  // ceil(2^40 / S): exact x / S for 0 <= x < 2^30, S <= 256
  __device__ __forceinline__ int div_S(int x) const { return (int)(((unsigned long long)(uint32_t)x * div_magic) >> 40); }
  __device__ __forceinline__ int slice_chunks(int sl) const { return sl < nchunks ? div_S(nchunks - 1 - sl) + 1 : 0; }
  __device__ __forceinline__ int slice_elems(int sl) const {
    const int c = slice_chunks(sl);
    if (c == 0) return 0;
    const int last = (c - 1) * S + sl;
    const int64_t rest = n - (int64_t)last * chunk_elems;
    return (c - 1) * chunk_elems + (int)(rest < chunk_elems ? rest : chunk_elems);
  }
  // local position in the slice buffer -> column of the row
  __device__ __forceinline__ int64_t column(int sl, int q) const {
    const int lc = q >> chunk_shift;
    return ((int64_t)(lc * S + sl) << chunk_shift) + (q & (chunk_elems - 1));
  }
};

// ---- bringing a slice into shared memory -------------------------------------------------
// Issued by warp 0 only.  TMA mode: one bulk copy per chunk, completion counted on `bar`;
// a ragged tail shorter than 16 bytes is copied with plain loads.  Otherwise (rows not
// 16-byte aligned) the warp copies the slice element by element and arrives on the barrier
// with a zero-byte expectation, so that waiting works the same way in both modes.
template <int DT>
__device__ __forceinline__ void issue_slice_load(const SampleParams& p, const Geometry& g, int64_t row, int sl,
                                                 unsigned char* buf, unsigned long long* bar) {
  using T = typename Elem<DT>::type;
  const T* src = reinterpret_cast<const T*>(p.logits) + row * p.row_stride;
  const int chunks = g.slice_chunks(sl);
  const int elems = g.slice_elems(sl);
  const int lane = lane_id();
  if (p.use_tma) {
    const uint32_t bytes = (uint32_t)elems * sizeof(T);
    const uint32_t bulk_bytes = bytes & ~15u;
    if (lane == 0) mbar_expect_tx(bar, bulk_bytes);
    __syncwarp();
    for (int lc = lane; lc < chunks; lc += 32) {
      uint32_t sz = kChunkBytes;
      if (lc == chunks - 1) sz = bulk_bytes - (uint32_t)lc * kChunkBytes;
      if (sz) bulk_load(buf + (size_t)lc * kChunkBytes, src + (int64_t)(lc * g.S + sl) * g.chunk_elems, sz, bar);
    }
    // ragged tail of the row's last chunk (fewer than 16 bytes)
    const int tail_first = (int)(bulk_bytes / sizeof(T));
    for (int q = tail_first + lane; q < elems; q += 32) reinterpret_cast<T*>(buf)[q] = src[g.column(sl, q)];
  } else {
    for (int q = lane; q < elems; q += 32) reinterpret_cast<T*>(buf)[q] = src[g.column(sl, q)];
    __syncwarp();
    if (lane == 0) mbar_expect_tx(bar, 0);
  }
}

// Calls f(value, local position) for every element of a slice buffer, 16-byte loads.
template <int DT, typename F>
__device__ __forceinline__ void for_each_slice_elem(const unsigned char* buf, int elems, F&& f) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  const int nvec = elems / VEC;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = vp[i];
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) f(e[j], i * VEC + j);
  }
  for (int q = nvec * VEC + threadIdx.x; q < elems; q += blockDim.x) f(reinterpret_cast<const T*>(buf)[q], q);
}

__device__ __forceinline__ SliceHeader* record_header(const SampleParams& p, int64_t row, int sl) {
  return reinterpret_cast<SliceHeader*>(p.records + ((size_t)row * p.S + sl) * kRecordBytes);
}
__device__ __forceinline__ unsigned char* record_payload(const SampleParams& p, int64_t row, int sl) {
  return p.records + ((size_t)row * p.S + sl) * kRecordBytes + sizeof(SliceHeader);
}

// ---- slice reducers -----------------------------------------------------------------------
// The greedy and candidate reducers are warp-local: every warp works on the vectors its lanes
// own (thread t owns the 16-byte vectors t, t + blockDim, ...) and leaves its result in the
// Control block; no block-wide barrier is needed until the slice is published.
__device__ __forceinline__ __nv_bfloat162 bf162_bits(uint32_t w) {
  __nv_bfloat162 r;
  memcpy(&r, &w, sizeof(r));
  return r;
}

// Block-wide max / min of one u32 per thread: one redux per warp, one shared-memory round.
__device__ __forceinline__ uint32_t block_max_u32(uint32_t v, uint32_t* scratch) {
  v = __reduce_max_sync(0xFFFFFFFFu, v);
  if (lane_id() == 0) scratch[warp_id()] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  uint32_t r = __reduce_max_sync(0xFFFFFFFFu, scratch[lane_id() < nw ? lane_id() : 0]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ uint32_t block_min_u32(uint32_t v, uint32_t* scratch) {
  return ~block_max_u32(~v, scratch);
}

// Largest key among the thread's first `vecs` vectors of a slice (all of them when vecs is
// large), 0 if it owns none.  bf16 uses packed NaN-propagating maxima; the key is only formed
// once at the end.
template <int DT>
__device__ __forceinline__ uint32_t thread_max_key(const unsigned char* buf, int nvec, int vecs) {
  using T = typename Elem<DT>::type;
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  if constexpr (DT == TLX_BF16) {
    __nv_bfloat162 mx = __float2bfloat162_rn(-INFINITY);
    bool any = false;
    for (int j = 0, i = threadIdx.x; j < vecs && i < nvec; ++j, i += blockDim.x) {
      const uint4 v = vp[i];
      mx = __hmax2_nan(__hmax2_nan(mx, bf162_bits(v.x)),
                       __hmax2_nan(bf162_bits(v.y), __hmax2_nan(bf162_bits(v.z), bf162_bits(v.w))));
      any = true;
    }
    if (!any) return 0u;
    const uint32_t kl = f32_key(__low2float(mx)), kh = f32_key(__high2float(mx));
    return kl > kh ? kl : kh;
  } else {
    constexpr int VEC = 16 / (int)sizeof(T);
    uint32_t mk = 0;
    for (int j = 0, i = threadIdx.x; j < vecs && i < nvec; ++j, i += blockDim.x) {
      const uint4 v = vp[i];
      T e[VEC];
      memcpy(e, &v, sizeof(v));
#pragma unroll
      for (int t = 0; t < VEC; ++t) { const uint32_t k = Elem<DT>::key(e[t]); mk = k > mk ? k : mk; }
    }
    return mk;
  }
}

template <int DT>
__device__ __forceinline__ typename Elem<DT>::type slice_elem(const unsigned char* buf, int q) {
  return reinterpret_cast<const typename Elem<DT>::type*>(buf)[q];
}

// Threshold bin from one bin per thread: the largest 12-bit bin B such that at least `want`
// threads have a bin >= B.  One block-wide vote per bit; threads without data vote with -1.
__device__ __forceinline__ int vote_threshold_bin(int my_bin, int want) {
  int lo = 0;
#pragma unroll
  for (int bit = 11; bit >= 0; --bit) {
    const int mid = lo | (1 << bit);
    if (__syncthreads_count(my_bin >= mid) >= want) lo = mid;
  }
  return lo;
}

// The same over 16-bit keys (the top halves of the 32-bit keys): 16 votes.
__device__ __forceinline__ int vote_threshold_key16(int my_key16, int want) {
  int lo = 0;
#pragma unroll
  for (int bit = 15; bit >= 0; --bit) {
    const int mid = lo | (1 << bit);
    if (__syncthreads_count(my_key16 >= mid) >= want) lo = mid;
  }
  return lo;
}

// A float that no element with key >= `key` is below (never a NaN pattern): the packed compares
// screen with it, the exact test is on the keys.
__device__ __forceinline__ float key_lower_value(uint32_t key) {
  const uint32_t b = key >> kHistShift;
  if (b <= 7) return -INFINITY;   // -inf itself lives in bin 7
  if (b >= 4088) key = 4088u << kHistShift;
  return key_f32(key);
}

// Greedy row: this warp's arg-max as key << 32 | (0x7FFFFFFF - local position); positions
// grow with the column inside a slice, so the lowest position is the lowest column.
template <int DT>
__device__ __forceinline__ void reduce_slice_greedy(const unsigned char* buf, int elems, WarpResults& wr) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  const int nvec = elems / VEC;
  uint32_t tkey = thread_max_key<DT>(buf, nvec, 1 << 30);
  for (int q = nvec * VEC + threadIdx.x; q < elems; q += blockDim.x) {   // ragged tail of the row's last slice
    const uint32_t k = Elem<DT>::key(slice_elem<DT>(buf, q));
    tkey = k > tkey ? k : tkey;
  }
  const uint32_t wkey = __reduce_max_sync(0xFFFFFFFFu, tkey);
  uint32_t qmin = 0xFFFFFFFFu;
  if (tkey == wkey) {   // only the lanes that hold the warp's maximum look for its first position
    const uint4* vp = reinterpret_cast<const uint4*>(buf);
    for (int i = threadIdx.x; i < nvec && qmin == 0xFFFFFFFFu; i += blockDim.x) {
      bool here = true;
      if constexpr (DT == TLX_BF16) {
        if (wkey != 0xFFFFFFFFu) {   // packed equality screens the vector (-0 == +0, as in the key domain)
          const uint4 v = vp[i];
          const __nv_bfloat162 m2 = __float2bfloat162_rn(key_f32(wkey));
          here = (__heq2_mask(bf162_bits(v.x), m2) | __heq2_mask(bf162_bits(v.y), m2) |
                  __heq2_mask(bf162_bits(v.z), m2) | __heq2_mask(bf162_bits(v.w), m2)) != 0u;
        }
      }
      if (here) {
#pragma unroll
        for (int t = VEC - 1; t >= 0; --t)
          if (Elem<DT>::key(slice_elem<DT>(buf, i * VEC + t)) == wkey) qmin = (uint32_t)(i * VEC + t);
      }
    }
    for (int q = nvec * VEC + threadIdx.x; q < elems; q += blockDim.x)
      if (Elem<DT>::key(slice_elem<DT>(buf, q)) == wkey && (uint32_t)q < qmin) qmin = (uint32_t)q;
  }
  qmin = __reduce_min_sync(0xFFFFFFFFu, qmin);
  if (lane_id() == 0)
    wr.top[warp_id()] = qmin == 0xFFFFFFFFu ? 0ull : ((unsigned long long)wkey << 32) | (uint32_t)(0x7FFFFFFF - (int)qmin);
}

// Row with 1 <= top_k <= kFastK: this warp publishes every element of its vectors at or above
// a warp-local threshold bin into its own segment of the slice record.  The bin is estimated
// so that about 2 m elements of the slice pass, m = K/S + 6 sqrt(K/S) + 8: each lane takes the
// maximum of a few of its elements and the bin is read off the distribution of those maxima
// (the chance that a lane's e elements contain one of the top fraction f is 1 - (1 - f)^e).
// A poor estimate costs time, never correctness: the merge checks that enough candidates lie
// above the highest threshold used.  `hits` is this warp's scratch list (kWarpHits entries).
template <int DT>
__device__ __forceinline__ void reduce_slice_fast(const Geometry& g, int sl, int K, const unsigned char* buf, int elems,
                                                  uint64_t* out_segment, unsigned short* hits, WarpResults& wr) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  const int lane = lane_id(), w = warp_id();
  const uint32_t lt_mask = (1u << lane) - 1u;
  const float share = (float)K / (float)g.S;
  const float m = share + 6.f * sqrtf(share) + 8.f;
  const float frac = fminf(1.f, 2.f * m / (float)(elems > 0 ? elems : 1));  // fraction of the slice that should pass
  const int nvec = elems / VEC;
  const int vec_per_thread = (nvec + (int)blockDim.x - 1) / (int)blockDim.x;
  int vecs = (int)(0.7f / (frac * VEC) + 0.5f);   // keep frac * (elements looked at) around 0.7 or below
  vecs = vecs < 1 ? 1 : (vecs > vec_per_thread ? vec_per_thread : vecs);
  const float p_lane = 1.f - __expf((float)(vecs * VEC) * __logf(fmaxf(1.f - frac, 1e-6f)));

  const uint32_t tkey = thread_max_key<DT>(buf, nvec, vecs);
  const bool has = (int)threadIdx.x < nvec;
  const int my_bin = has ? (int)(tkey >> kHistShift) : -1;
  const int holders = __popc(__ballot_sync(0xFFFFFFFFu, has));
  int want = (int)((float)holders * p_lane + 0.999f);
  want = want < 1 ? 1 : want;
  int bin = 0;   // largest bin such that at least `want` lanes have a maximum at or above it
#pragma unroll
  for (int bit = 11; bit >= 0; --bit) {
    const int mid = bin | (1 << bit);
    if (__popc(__ballot_sync(0xFFFFFFFFu, my_bin >= mid)) >= want) bin = mid;
  }
  // One threshold for the whole slice: the lower quartile of the warps' estimates (a single
  // warp's estimate is noisy, and the merge can only use the highest threshold of a row).
  if (lane == 0) wr.bin[w] = holders ? (unsigned short)bin : (unsigned short)0xFFFF;
  __syncthreads();
  {
    const int nw = (int)blockDim.x >> 5;
    const int j = lane % nw;
    const uint32_t mine = wr.bin[j];
    int rank = 0, live = 0;
    for (int t = 0; t < nw; ++t) {
      const uint32_t other = wr.bin[t];
      live += other != 0xFFFFu;
      rank += (other < mine || (other == mine && t < j)) ? 1 : 0;
    }
    const uint32_t pick = __ballot_sync(0xFFFFFFFFu, lane < nw && rank == live / 4);
    bin = pick ? (int)__shfl_sync(0xFFFFFFFFu, mine, __ffs(pick) - 1) : 0;
    if (bin == 0xFFFF) bin = 0;
  }
  const uint32_t min_key = (uint32_t)bin << kHistShift;

  // step 1: which of this warp's vectors hold an element at or above the threshold
  int nhits = 0;
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  const float thr = bin_lower_value(bin);
  const __nv_bfloat162 thr2 = __float2bfloat162_rn(thr);   // bin edges are exact in bf16
  for (int i0 = w * 32; i0 < nvec; i0 += blockDim.x) {
    const int i = i0 + lane;
    bool hit = false;
    if (i < nvec) {
      const uint4 v = vp[i];
      if constexpr (DT == TLX_BF16) {
        // __hblt2: both halves ordered and below the threshold (a NaN fails it and is looked at)
        hit = !(__hblt2(bf162_bits(v.x), thr2) && __hblt2(bf162_bits(v.y), thr2) && __hblt2(bf162_bits(v.z), thr2) &&
                __hblt2(bf162_bits(v.w), thr2));
      } else {
        hit = !(__uint_as_float(v.x) < thr && __uint_as_float(v.y) < thr && __uint_as_float(v.z) < thr &&
                __uint_as_float(v.w) < thr);
      }
    }
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, hit);
    if (hit) hits[nhits + __popc(mask & lt_mask)] = (unsigned short)i;
    nhits += __popc(mask);
  }
  __syncwarp();
  // step 2: expand the noted vectors densely and publish what passes
  int count = 0;
  auto offer = [&](bool valid, int q) {
    uint32_t key = 0;
    bool pass = false;
    if (valid) {
      key = Elem<DT>::key(slice_elem<DT>(buf, q));
      pass = key >= min_key;
    }
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, pass);
    if (pass) {
      const int pos = count + __popc(mask & lt_mask);
      if (pos < kWarpCap) out_segment[pos] = cand_make(key, (uint32_t)g.column(sl, q));
    }
    count += __popc(mask);
  };
  for (int e0 = 0; e0 < nhits * VEC; e0 += 32) {
    const int e = e0 + lane;
    const bool valid = e < nhits * VEC;
    offer(valid, valid ? (int)hits[e / VEC] * VEC + (e % VEC) : 0);
  }
  if (w == 0)   // ragged tail of the row's last slice (fewer than VEC elements)
    for (int q0 = nvec * VEC; q0 < elems; q0 += 32) offer(q0 + lane < elems, q0 + lane);
  if (lane == 0) {
    wr.count[w] = (unsigned short)(count < kWarpCap ? count : kWarpCap);
    wr.overflow[w] = count > kWarpCap ? 1 : 0;
    if (w == 0) wr.cutoff_bin = bin;
  }
}

// bf16 row without a small top-k: slice maximum, full-key histogram of the kWin keys below it
// (published as 16-bit counts: a slice holds fewer than 65536 elements), and the sum of
// exp(x - slice max) over the elements BELOW that window.  The softmax mass of a histogram bin
// is count * exp(value - max), so the merge gets the exact mass of everything in the window
// from the counts.  `win` is the CTA's kWin-bin area.
__device__ __forceinline__ void reduce_slice_general_bf16(const SampleParams& p, const Geometry& g, int64_t row,
                                                          int sl, const unsigned char* buf, int elems,
                                                          SelectShared& s, uint32_t* win) {
  SliceHeader* hdr = record_header(p, row, sl);
  uint32_t* out = reinterpret_cast<uint32_t*>(record_payload(p, row, sl));
  const int nvec = elems / 8;
  uint32_t tkey = thread_max_key<TLX_BF16>(buf, nvec, 1 << 30);
  for (int q = nvec * 8 + threadIdx.x; q < elems; q += blockDim.x) {
    const uint32_t k = Elem<TLX_BF16>::key(slice_elem<TLX_BF16>(buf, q));
    tkey = k > tkey ? k : tkey;
  }
  const uint32_t kmax32 = block_max_u32(tkey, s.scan_u32);
  const int kmax = (int)(kmax32 >> 16);
  const float smax = key_f32(kmax32);
  for (int i = threadIdx.x; i < kWin; i += blockDim.x) win[i] = 0;
  __syncthreads();
  // One element = 16 raw bits h.  Its 16-bit key is h + 0x8000 for a cleared sign and 0xFFFF - h
  // otherwise; its histogram slot is kmax - key if that is inside the window, else exp(x - max)
  // goes to the below-window sum.  (-0 keeps its own slot next to +0: same value, same mass.)
  const float neg_smax_l2e = -smax * 1.44269504f;
  float below = 0.f;
  auto ex2 = [](float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; };
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  if (kmax >= 0x8000 + kWin) {
    // positive maximum (the usual case): every negative element is below the window, and one
    // unsigned compare of (kmax - 0x8000) - h against the window size decides
    const uint32_t dpos = (uint32_t)(kmax - 0x8000);
    auto visit = [&](uint32_t h, float x) {
      const uint32_t d = dpos - h;
      const float e = ex2(fmaf(x, 1.44269504f, neg_smax_l2e));
      if (d < (uint32_t)kWin) atomicAdd(&win[d], 1u);
      else below += e;
    };
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 v = vp[i];
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        visit(w4[j] & 0xFFFFu, __uint_as_float(w4[j] << 16));
        visit(w4[j] >> 16, __uint_as_float(w4[j] & 0xFFFF0000u));
      }
    }
    for (int q = nvec * 8 + threadIdx.x; q < elems; q += blockDim.x) {
      const uint32_t h = reinterpret_cast<const unsigned short*>(buf)[q];
      visit(h, __uint_as_float(h << 16));
    }
  } else {
    auto visit = [&](uint32_t h) {
      const uint32_t k16 = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);
      const int d = kmax - (int)k16;
      const float e = ex2(fmaf(__uint_as_float(h << 16), 1.44269504f, neg_smax_l2e));
      if (d >= 0 && d < kWin) atomicAdd(&win[d], 1u);
      else if (d >= kWin) below += e;
    };
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 v = vp[i];
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { visit(w4[j] & 0xFFFFu); visit(w4[j] >> 16); }
    }
    for (int q = nvec * 8 + threadIdx.x; q < elems; q += blockDim.x)
      visit((uint32_t)reinterpret_cast<const unsigned short*>(buf)[q]);
  }
  double total;
  block_scan_incl<double>((double)below, s.scan_f64, &total, ShflUpF64());
  for (int i = threadIdx.x; i < kWin / 2; i += blockDim.x) out[i] = win[2 * i] | (win[2 * i + 1] << 16);
  if (threadIdx.x == 0) {
    hdr->kmax16 = kmax;
    hdr->smax = smax;
    hdr->mass = total;
    hdr->top = ((unsigned long long)kmax32 << 32) | 1ull;
  }
}

// Finds the elements of a tile whose key is >= min_key and hands them to `sink`.  `thr` is a
// float (exactly representable in the tile's dtype) such that every element with key >= min_key
// satisfies !(x < thr).  Warp-local in two steps: a packed compare notes the (few) elements that
// may pass, then those are looked at densely, so that a rare passing element does not drag its
// whole warp through the slow path.  `hits` is this warp's scratch list of local positions.
// sink(pass, key, q) is called by all 32 lanes together (pass == false for lanes without one).
template <int DT, typename Sink>
__device__ __forceinline__ void scan_tile(const unsigned char* buf, int elems, float thr, uint32_t min_key,
                                          unsigned short* hits, Sink&& sink) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int kHitCap = kHistBins * 2 / kWarps;   // the idle histogram holds the warps' lists (u16 entries)
  const int lane = lane_id(), w = warp_id();
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int nvec = elems / VEC;
  const __nv_bfloat162 thr2 = __float2bfloat162_rn(thr);
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  int nhits = 0;
  // step 1: per vector, a coarse test (may anything in it pass?) and, only where it says yes, a bit
  // mask of the elements that are not (ordered and) below the threshold.  The coarse answers of a
  // round are put to one warp vote, so that the usual round without any hit is a handful of
  // instructions behind a warp-uniform branch.
  auto coarse = [&](const uint4& v) -> bool {
    if constexpr (DT == TLX_BF16) {
      const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(v.x), bf162_bits(v.y)),
                                           __hmax2_nan(bf162_bits(v.z), bf162_bits(v.w)));
      return !__hblt2(m, thr2);
    } else {
      return !(__uint_as_float(v.x) < thr) || !(__uint_as_float(v.y) < thr) || !(__uint_as_float(v.z) < thr) ||
             !(__uint_as_float(v.w) < thr);
    }
  };
  auto fine = [&](const uint4& v) -> uint32_t {
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
    uint32_t bits = 0;
    if constexpr (DT == TLX_BF16) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t below = __hlt2_mask(bf162_bits(w4[j]), thr2);   // 0xFFFF per half that is below
        bits |= ((below & 0xFFFFu) ? 0u : 1u) << (2 * j);
        bits |= ((below >> 16) ? 0u : 1u) << (2 * j + 1);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) bits |= (__uint_as_float(w4[j]) < thr ? 0u : 1u) << j;
    }
    return bits;
  };
  // step 2: the noted elements, densely
  auto offer = [&](bool valid, int q) {
    uint32_t key = 0;
    bool pass = false;
    if (valid) {
      key = Elem<DT>::key(slice_elem<DT>(buf, q));
      pass = key >= min_key;
    }
    sink(pass, key, q);
  };
  auto flush = [&]() {
    __syncwarp();
    for (int e0 = 0; e0 < nhits; e0 += 32) offer(e0 + lane < nhits, e0 + lane < nhits ? (int)hits[e0 + lane] : 0);
    __syncwarp();
    nhits = 0;
  };
  constexpr int kRound = 4;   // vectors per lane and round
  for (int base = w * 32; base < nvec; base += kRound * (int)blockDim.x) {
    uint4 v[kRound];
    bool maybe[kRound];
    bool any = false;
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      const int i = base + u * (int)blockDim.x + lane;
      v[u] = i < nvec ? vp[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      maybe[u] = (base + u * (int)blockDim.x + lane < nvec) && coarse(v[u]);
      any |= maybe[u];
    }
    const bool go = __any_sync(0xFFFFFFFFu, any);
    if (!go) continue;
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      const int i = base + u * (int)blockDim.x + lane;
      uint32_t bits = maybe[u] ? fine(v[u]) : 0u;
      while (__any_sync(0xFFFFFFFFu, bits != 0u)) {   // one element per lane and turn
        const bool have = bits != 0u;
        const uint32_t mask = __ballot_sync(0xFFFFFFFFu, have);
        if (have) {
          const int t = __ffs(bits) - 1;
          bits &= bits - 1;
          hits[nhits + __popc(mask & lt_mask)] = (unsigned short)(i * VEC + t);
        }
        nhits += __popc(mask);
      }
      if (nhits > kHitCap - 32 * VEC) flush();   // room for one more vector per lane
    }
  }
  flush();
  if (w == 0)   // ragged tail of the row's last tile (fewer than VEC elements)
    for (int q0 = nvec * VEC; q0 < elems; q0 += 32) offer(q0 + lane < elems, q0 + lane);
}

// Appends every element of the tile at or above bin `bin` to the candidate list; `col_of(q)`
// maps a local position to its column.  Warp-local in two steps.  Step 1: every lane brings in
// four vectors and puts one packed question to each (may anything in it pass?); the answers go
// to a single warp vote, and the usual round, without any such vector, ends there.  Otherwise the
// indices of those vectors are noted in the warp's list `hits`.  Step 2, once per tile: the
// listed vectors are looked at densely, one element per lane.
template <int DT, int WARPS, typename ColOf>
__device__ __forceinline__ void collect_tile(const unsigned char* buf, int elems, uint32_t min_key, SelectShared& s,
                                             uint64_t* cand, unsigned short* hits, ColOf col_of) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int kHitCap = kHistBins * 2 / WARPS;    // the idle histogram holds the warps' lists (u16 entries)
  constexpr int kRound = 4;                         // vectors per lane and round
  constexpr int kPerStep = 32 / VEC;                // listed vectors one step of the dense pass covers
  const float thr = key_lower_value(min_key);
  const int nvec = elems / VEC;
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  const int lane = lane_id(), w = warp_id();
  const uint32_t lt_mask = (1u << lane) - 1u;
  const __nv_bfloat162 thr2 = __float2bfloat162_rn(thr);
  int noted = 0;
  // Dense pass over listed positions, kSteps * 32 at a time: all loads first, then all votes, one
  // reservation in the candidate list, then the stores, so that the steps' latencies overlap.
  constexpr int kSteps = 4;
  auto offer_batch = [&](const bool (&valid)[kSteps], const int (&q)[kSteps]) {
    uint32_t key[kSteps], mask[kSteps];
    int total = 0;
#pragma unroll
    for (int j = 0; j < kSteps; ++j) key[j] = valid[j] ? Elem<DT>::key(slice_elem<DT>(buf, q[j])) : 0u;
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
      mask[j] = __ballot_sync(0xFFFFFFFFu, valid[j] && key[j] >= min_key);
      total += __popc(mask[j]);
    }
    if (total == 0) return;
    int run = 0;
    if (lane == 0) run = atomicAdd(&s.fill, total);
    run = __shfl_sync(0xFFFFFFFFu, run, 0);
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
      if (mask[j] & (1u << lane)) {
        const int pos = run + __popc(mask[j] & lt_mask);
        if (pos < kMergeCap) cand[pos] = cand_make(key[j], (uint32_t)col_of(q[j]));
      }
      run += __popc(mask[j]);
    }
  };
  auto flush = [&]() {
    __syncwarp();
    for (int k = 0; k < noted; k += kSteps * kPerStep) {
      bool valid[kSteps];
      int q[kSteps];
#pragma unroll
      for (int j = 0; j < kSteps; ++j) {
        const int slot = k + j * kPerStep + lane / VEC;
        valid[j] = slot < noted;
        q[j] = valid[j] ? (int)hits[slot] * VEC + (lane % VEC) : 0;
      }
      offer_batch(valid, q);
    }
    __syncwarp();
    noted = 0;
  };
  for (int base = w * 32; base < nvec; base += kRound * (int)blockDim.x) {
    uint4 v[kRound];
    bool maybe[kRound];
    bool any = false;
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      const int i = base + u * (int)blockDim.x + lane;
      v[u] = i < nvec ? vp[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      const bool inside = base + u * (int)blockDim.x + lane < nvec;
      if constexpr (DT == TLX_BF16) {
        const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(v[u].x), bf162_bits(v[u].y)),
                                             __hmax2_nan(bf162_bits(v[u].z), bf162_bits(v[u].w)));
        maybe[u] = inside && !__hblt2(m, thr2);
      } else {
        maybe[u] = inside && (!(__uint_as_float(v[u].x) < thr) || !(__uint_as_float(v[u].y) < thr) ||
                              !(__uint_as_float(v[u].z) < thr) || !(__uint_as_float(v[u].w) < thr));
      }
      any |= maybe[u];
    }
    const bool go = __any_sync(0xFFFFFFFFu, any);
    if (!go) continue;
#pragma unroll
    for (int u = 0; u < kRound; ++u) {
      const uint32_t mask = __ballot_sync(0xFFFFFFFFu, maybe[u]);
      if (maybe[u]) hits[noted + __popc(mask & lt_mask)] = (unsigned short)(base + u * (int)blockDim.x + lane);
      noted += __popc(mask);
    }
    if (noted > kHitCap - kRound * 32) flush();
  }
  flush();
  if (w == 0 && nvec * VEC < elems) {   // ragged end of the row's last tile (fewer than VEC elements)
    bool valid[kSteps];
    int q[kSteps];
#pragma unroll
    for (int j = 0; j < kSteps; ++j) { valid[j] = j == 0 && nvec * VEC + lane < elems; q[j] = nvec * VEC + lane; }
    offer_batch(valid, q);
  }
}

// Raises the threshold bin to the largest one that still has K candidates at or above it and
// drops the candidates below it.  The histogram is rebuilt from the list (it is not kept up
// to date while collecting).  All threads call.
static __device__ __noinline__ void refine_candidates(SelectShared& s, uint64_t* cand, int K) {
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) s.hist[i] = 0;
  __syncthreads();
  const int m = s.fill < kMergeCap ? s.fill : kMergeCap;
  for (int i = threadIdx.x; i < m; i += blockDim.x) atomicAdd(&s.hist[cand_key(cand[i]) >> kHistShift], 1u);
  const int old_bin = s.bin;
  __syncthreads();
  find_threshold_bin(s, K, old_bin);
  if (s.bin != old_bin) compact_candidates<kMergeCap>(s, cand);
  __syncthreads();
}

// Final pass over one slice of a row without top-k: every element with key >= the row's
// threshold gets its Gumbel score; the slice's winner (decided on the f64-evaluated Gumbel term
// among the contenders, as in final_argmax) is folded into the row's state with an atomic max,
// and the CTA that delivers the row's last slice writes the token.
__device__ __forceinline__ void reduce_slice_final_bf16(const SampleParams& p, const Geometry& g, int64_t row, int sl,
                                                        const unsigned char* buf, int elems, SelectShared& s,
                                                        unsigned char* uni) {
  RowState* rs = p.rowstate + row;
  const uint32_t min_key = rs->min_key;
  const float thr = rs->thr;
  const float T_ = p.temperature[row];
  const int64_t nrow = row + p.dim0_offset;
  unsigned short* hits = reinterpret_cast<unsigned short*>(s.hist) + warp_id() * (kHistBins * 2 / kWarps);
  constexpr int kListCap = (int)(kUnionBytes / 8) / kWarps;
  constexpr int kListPer = kListCap / 32;
  uint2* wlist = reinterpret_cast<uint2*>(uni) + warp_id() * kListCap;
  const uint32_t lt_mask = (1u << lane_id()) - 1u;
  const float inv_T = 1.0f / T_;
  float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
  uint32_t k1 = 0;
  int c1 = 0x7FFFFFFF;
  int wcount = 0;
  auto score_list = [&](float cut, Best* exact) {
    __syncwarp();
    float uu[kListPer];
#pragma unroll
    for (int j = 0; j < kListPer; ++j) {
      const int e = lane_id() + 32 * j;
      uu[j] = e < wcount ? p.noise.at(nrow, (int64_t)wlist[e].x) : 0.5f;
    }
#pragma unroll
    for (int j = 0; j < kListPer; ++j) {
      const int e = lane_id() + 32 * j;
      if (e < wcount) {
        // screening score: reciprocal instead of the division, fast logs (both well inside the slack)
        const float a = key_f32(wlist[e].y) * inv_T + gumbel_screen(uu[j]);
        if (exact) {
          if (a >= cut)
            *exact = best_of(*exact, Best{__fdiv_rn(key_f32(wlist[e].y), T_) + gumbel_exact(uu[j]), (int)wlist[e].x});
        } else if (a > a1) { a2 = a1; a1 = a; k1 = wlist[e].y; u1 = uu[j]; c1 = (int)wlist[e].x; }
        else if (a > a2) a2 = a;
      }
    }
    __syncwarp();
    wcount = 0;
  };
  auto scan = [&](float cut, Best* exact) {
    scan_tile<TLX_BF16>(buf, elems, thr, min_key, hits, [&](bool pass, uint32_t key, int q) {
      const uint32_t mask = __ballot_sync(0xFFFFFFFFu, pass);
      if (pass) wlist[wcount + __popc(mask & lt_mask)] = make_uint2((uint32_t)g.column(sl, q), key);
      wcount += __popc(mask);
      if (wcount > kListCap - 32) score_list(cut, exact);
    });
    score_list(cut, exact);
  };
  scan(0.f, nullptr);
  const Best top = block_best(Best{a1, c1}, s);
  const float cut = top.y - (kGumbelSlack + 1e-5f * fabsf(top.y));
  Best best{-INFINITY, 0x7FFFFFFF};
  if (__syncthreads_or(a2 >= cut)) {
    scan(cut, &best);   // a thread saw two contenders: look at the slice again and decide exactly
  } else if (a1 >= cut) {
    best = Best{__fdiv_rn(key_f32(k1), T_) + gumbel_exact(u1), c1};
  }
  best = block_best(best, s);
  if (threadIdx.x == 0 && best.tok != 0x7FFFFFFF) {
    const unsigned long long packed = ((unsigned long long)f32_key(best.y) << 32) | (uint32_t)(0x7FFFFFFF - best.tok);
    atomicMax(&rs->best, packed);
  }
}

// ---- row merges (run by the CTA that completed the row's last slice) ------------------------
template <typename T>
__device__ __forceinline__ T ld_cg(const T* p) { return __ldcg(p); }

static __device__ __noinline__ int merge_row_greedy(const SampleParams& p, int64_t row, SelectShared& s) {
  uint64_t best = 0;
  if ((int)threadIdx.x < p.S) best = ld_cg(&record_header(p, row, threadIdx.x)->top);
  block_max_u64(best, s);
  return 0x7FFFFFFF - (int32_t)(uint32_t)best;
}

// Gathers the published candidates of a row that lie at or above the highest slice threshold
// into cand[]; returns their number, or -1 if the published sets cannot be trusted to hold
// the row's top-K (a segment overflowed, or fewer than K candidates).  A row's candidates
// sit in S * kWarps segments (one per slice and publishing warp).
static __device__ __noinline__ int gather_candidates(const SampleParams& p, int64_t row, int K, SelectShared& s,
                                                 uint64_t* cand) {
  if (threadIdx.x == 0) { s.tmp_i[0] = 0; s.tmp_i[1] = 0; s.fill = 0; }
  __syncthreads();
  const int nseg = p.S * kWarps;
  uint32_t carry = 0;
  for (int base = 0; base < nseg; base += blockDim.x) {
    const int seg = base + threadIdx.x;
    uint32_t cnt = 0;
    if (seg < nseg) {
      const SliceHeader* h = record_header(p, row, seg / kWarps);
      cnt = ld_cg(&h->wcount[seg % kWarps]);
      if (seg % kWarps == 0) {
        atomicMax(&s.tmp_i[0], ld_cg(&h->cutoff_bin));
        if (ld_cg(&h->overflow)) atomicOr(&s.tmp_i[1], 1);
      }
    }
    uint32_t total;
    const uint32_t incl = block_scan_incl<uint32_t>(cnt, s.scan_u32, &total, ShflUpU32());
    if (seg < nseg) s.hist[seg] = carry + incl;   // inclusive offsets of the segments
    carry += total;
  }
  __syncthreads();
  if (s.tmp_i[1] != 0) return -1;
  const uint32_t min_key = (uint32_t)s.tmp_i[0] << kHistShift;
  for (uint32_t f = threadIdx.x; f < carry; f += blockDim.x) {
    int lo = 0, hi = nseg - 1;   // first segment whose inclusive offset exceeds f
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s.hist[mid] > f) hi = mid; else lo = mid + 1;
    }
    const uint32_t before = lo ? s.hist[lo - 1] : 0u;
    const uint64_t* seg_base =
        reinterpret_cast<const uint64_t*>(record_payload(p, row, lo / kWarps)) + (lo % kWarps) * kWarpCap;
    const uint64_t c = ld_cg(seg_base + (f - before));
    if (cand_key(c) >= min_key) {
      const int slot = atomicAdd(&s.fill, 1);
      if (slot < kMergeCap) cand[slot] = c;
    }
  }
  __syncthreads();
  const int m = s.fill;
  return (m > kMergeCap || m < K) ? -1 : m;
}

// Number of the `n` listed tokens below `tok`.
static __device__ __noinline__ uint32_t tie_rank(const uint32_t* tie_tok, int n, uint32_t tok) {
  uint32_t rank = 0;
  for (int j = 0; j < n; ++j) rank += tie_tok[j] < tok ? 1u : 0u;
  return rank;
}

// Sampler tail on unsorted bf16 candidates, without sorting them: a histogram over the
// candidates' 16-bit keys gives the top-k boundary (key and admitted ties), the softmax
// denominator and the top-p threshold exactly as in the whole-row path (the mass of a value
// group is count * exp(value - max)); the Gumbel arg-max then runs over the kept candidates.
// Needs the keys to span at most kHistBins values; returns -1 otherwise (caller sorts).
static __device__ __noinline__ int tail_bf16_hist(const SampleParams& p, int64_t row, int K, float pp, float T_, int m,
                                              SelectShared& s, const uint64_t* cand) {
  uint32_t kmx = 0, kmn = 0xFFFFFFFFu;
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    const uint32_t k16 = cand_key(cand[i]) >> 16;
    kmx = k16 > kmx ? k16 : kmx;
    kmn = k16 < kmn ? k16 : kmn;
  }
  const int kmax = (int)block_max_u32(kmx, s.scan_u32);
  const int kmin = (int)block_min_u32(kmn, s.scan_u32);
  const int W = kmax - kmin + 1;
  if (W > kHistBins) return -1;
  TLX_STAMP(p, 3);
  uint32_t* win = s.hist;   // win[kmax - key16]
  for (int i = threadIdx.x; i < W; i += blockDim.x) win[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < m; i += blockDim.x) atomicAdd(&win[kmax - (int)(cand_key(cand[i]) >> 16)], 1u);
  __syncthreads();
  const float xmax = key16_value(kmax);
  const int per = (W + (int)blockDim.x - 1) / (int)blockDim.x;
  const int i0 = threadIdx.x * per;

  // top-k boundary: first bin (descending key) at which the running count reaches K
  uint32_t local = 0;
  for (int j = 0; j < per; ++j) if (i0 + j < W) local += win[i0 + j];
  uint32_t total;
  const uint32_t incl = block_scan_incl<uint32_t>(local, s.scan_u32, &total, ShflUpU32());
  const uint32_t before = incl - local;
  if (before < (uint32_t)K && incl >= (uint32_t)K) {
    uint32_t run = before;
    for (int j = 0; j < per; ++j) {
      const uint32_t c = win[i0 + j];
      if (run + c >= (uint32_t)K) { s.tmp_i[0] = i0 + j; s.tmp_i[1] = (int)((uint32_t)K - run); s.tmp_i[2] = (int)c; break; }
      run += c;
    }
  }
  __syncthreads();
  const int vk_idx = s.tmp_i[0];
  const uint32_t ties_admitted = (uint32_t)s.tmp_i[1], ties_total = (uint32_t)s.tmp_i[2];
  TLX_STAMP(p, 4);
  // denominator and top-p threshold over the top-k set
  double mass = 0.0;
  for (int j = 0; j < per; ++j) {
    const int idx = i0 + j;
    if (idx < W && idx <= vk_idx) {
      const uint32_t c = idx == vk_idx ? ties_admitted : win[idx];
      if (c) mass += (double)c * (double)expf(key16_value(kmax - idx) - xmax);
    }
  }
  double Z;
  const double mincl = block_scan_incl<double>(mass, s.scan_f64, &Z, ShflUpF64());
  const double target = (double)pp * Z;
  if (threadIdx.x == 0) s.tmp_i[3] = vk_idx;   // default: keep the whole top-k set
  __syncthreads();
  if (mincl - mass < target && mincl >= target) {
    double run = mincl - mass;
    for (int j = 0; j < per; ++j) {
      const int idx = i0 + j;
      if (idx < W && idx <= vk_idx) {
        const uint32_t c = idx == vk_idx ? ties_admitted : win[idx];
        if (c) {
          run += (double)c * (double)expf(key16_value(kmax - idx) - xmax);
          if (run >= target) { s.tmp_i[3] = idx; break; }
        }
      }
    }
  }
  __syncthreads();
  const int vstar_idx = s.tmp_i[3];
  const bool cut_ties = vstar_idx == vk_idx && ties_admitted < ties_total;
  __syncthreads();
  TLX_STAMP(p, 5);
  // the lowest tokens of the boundary group are the admitted ones: list the group's tokens
  uint32_t* tie_tok = s.hist;   // the histogram is no longer needed
  if (cut_ties) {
    if (threadIdx.x == 0) s.fill = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
      const uint64_t c = cand[i];
      if (kmax - (int)(cand_key(c) >> 16) == vk_idx) tie_tok[atomicAdd(&s.fill, 1)] = cand_low(c);
    }
    __syncthreads();
  }
  const int n_ties = cut_ties ? s.fill : 0;
  // Gumbel arg-max over the kept candidates, screened in f32 (see final_argmax)
  const int64_t nrow = row + p.dim0_offset;
  float a1 = -INFINITY, a2 = -INFINITY, q1 = 0.f, u1 = 0.5f;
  int c1 = 0x7FFFFFFF;
  auto kept = [&](uint64_t c) {
    const int idx = kmax - (int)(cand_key(c) >> 16);
    if (idx > vstar_idx) return false;
    if (idx < vk_idx || !cut_ties) return true;
    // idx == vk_idx: admitted if fewer than ties_admitted group members have a lower token
    return tie_rank(tie_tok, n_ties, cand_low(c)) < ties_admitted;
  };
  {
    // decide which of the thread's candidates are kept and start their noise loads, four at a time
    constexpr int kBatch = 4;
#pragma unroll 1
    for (int i0b = threadIdx.x; i0b < m; i0b += kBatch * (int)blockDim.x) {
      uint32_t keep_mask = 0;
      float uu[kBatch];
      uint64_t cc[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int i = i0b + j * (int)blockDim.x;
        uu[j] = 0.5f;
        cc[j] = 0;
        if (i < m) {
          cc[j] = cand[i];
          if (kept(cc[j])) { keep_mask |= 1u << j; uu[j] = p.noise.at(nrow, (int64_t)cand_low(cc[j])); }
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (keep_mask & (1u << j)) {
          const float q = __fdiv_rn(key_f32(cand_key(cc[j])), T_);
          const float a = q + gumbel_screen(uu[j]);
          if (a > a1) { a2 = a1; a1 = a; q1 = q; u1 = uu[j]; c1 = (int)cand_low(cc[j]); }
          else if (a > a2) a2 = a;
        }
      }
    }
  }
  TLX_STAMP(p, 6);
  const Best top = block_best(Best{a1, c1}, s);
  const float cut = top.y - (kGumbelSlack + 1e-5f * fabsf(top.y));
  const int leaders = __syncthreads_count(a1 >= cut);
  const int crowded = __syncthreads_or(a2 >= cut);
  TLX_STAMP(p, 7);
  // nothing else comes within the slack of the best screened score: it is the winner as it stands
  if (leaders == 1 && !crowded) return top.tok;
  Best best{-INFINITY, 0x7FFFFFFF};
  if (!crowded) {
    if (a1 >= cut) best = Best{q1 + gumbel_exact(u1), c1};
  } else {
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
      const uint64_t c = cand[i];
      if (kept(c)) {
        const float u = p.noise.at(nrow, (int64_t)cand_low(c));
        const float q = __fdiv_rn(key_f32(cand_key(c)), T_);
        if (q + gumbel_screen(u) >= cut) best = best_of(best, Best{q + gumbel_exact(u), (int)cand_low(c)});
      }
    }
  }
  const int result = block_best(best, s).tok;
  return result;
}

template <int DT>
static __device__ __noinline__ int merge_row_fast(const SampleParams& p, int64_t row, int K, float pp, float T_,
                                              SelectShared& s, uint64_t* cand, int* status) {
  using T = typename Elem<DT>::type;
  const T* rowp = reinterpret_cast<const T*>(p.logits) + row * p.row_stride;
  int m = gather_candidates(p, row, K, s, cand);
  __syncthreads();
  if (m < 0) {
    exact_select_row<DT>(rowp, p.vocab, K, s, cand);
    m = K;
    *status |= kStatusRedone;
    __syncthreads();
  }
  if constexpr (DT == TLX_BF16) {
    const int tok = tail_bf16_hist(p, row, K, pp, T_, m, s, cand);
    if (tok >= 0) return tok;
    __syncthreads();
  }
  sort_candidates(cand, m);
  const int64_t nrow = row + p.dim0_offset;
  return sample_tail<2>(
      K, pp, T_, s, [&](int i) { return key_f32(cand_key(cand[i])); }, [&](int i) { return (int)cand_low(cand[i]); },
      [&](int i) { return p.noise.at(nrow, (int64_t)cand_low(cand[i])); });
}

static __device__ __noinline__ int merge_row_general_bf16(const SampleParams& p, int64_t row, int K, float pp, float T_,
                                                      SelectShared& s, uint32_t* win, bool threshold_only = false) {
  const __nv_bfloat16* rowp = reinterpret_cast<const __nv_bfloat16*>(p.logits) + row * p.row_stride;
  if (threadIdx.x == 0) s.tmp_i[0] = 0;
  for (int i = threadIdx.x; i < kWin; i += blockDim.x) win[i] = 0;
  __syncthreads();
  float smax = 0.f;
  double below = 0.0;
  if ((int)threadIdx.x < p.S) {
    const SliceHeader* h = record_header(p, row, threadIdx.x);
    const int k = ld_cg(&h->kmax16);
    s.hist[256 + threadIdx.x] = (uint32_t)k;
    atomicMax(&s.tmp_i[0], k);
    smax = ld_cg(&h->smax);
    below = ld_cg(&h->mass);
  }
  __syncthreads();
  const int kmax = s.tmp_i[0];
  const float xmax = key16_value(kmax);
  // mass below the row's window: the slices' below-window sums, rescaled to the row maximum ...
  double part = ((int)threadIdx.x < p.S) ? below * (double)expf(smax - xmax) : 0.0;
  // ... plus whatever of a slice's window hangs out below the row's.  The windows are added up
  // shifted by (row max - slice max); 16-byte loads, several in flight per thread.
  constexpr int kVecPerSlice = kWin / 8;   // 8 counts per 16-byte vector
  const int nv = p.S * kVecPerSlice;
  for (int v0 = threadIdx.x; v0 < nv; v0 += 4 * blockDim.x) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * blockDim.x;
      r[u] = make_uint4(0, 0, 0, 0);
      if (v < nv)
        r[u] = ld_cg(reinterpret_cast<const uint4*>(record_payload(p, row, v / kVecPerSlice)) + (v % kVecPerSlice));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * blockDim.x;
      if (v >= nv) continue;
      const int sl = v / kVecPerSlice;
      const int shift = kmax - (int)s.hist[256 + sl];
      const uint32_t w4[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t c = (j & 1) ? (w4[j >> 1] >> 16) : (w4[j >> 1] & 0xFFFFu);
        if (c) {
          const int idx = (v % kVecPerSlice) * 8 + j + shift;
          if (idx < kWin) atomicAdd(&win[idx], c);
          else if (kmax - idx >= 0) part += (double)c * (double)expf(key16_value(kmax - idx) - xmax);
        }
      }
    }
  }
  __syncthreads();
  // denominator over the whole row = mass inside the window (from the counts) + mass below it
  for (int i = threadIdx.x; i < kWin; i += blockDim.x) {
    const uint32_t c = win[i];
    if (c && kmax - i >= 0) part += (double)c * (double)expf(key16_value(kmax - i) - xmax);
  }
  double Z;
  block_scan_incl<double>(part, s.scan_f64, &Z, ShflUpF64());
  RowPreset pre;
  pre.top = ((uint64_t)key16_to_key32((uint32_t)kmax) << 32) | 1ull;
  pre.have_window = true;
  pre.mass = Z;
  pre.threshold_only = threshold_only;
  return general_row_bf16<kWin>(rowp, p.vocab, K, pp, T_, p.noise, row + p.dim0_offset, s, win, pre);
}

// class and effective top-k of a row, from global memory
__device__ __forceinline__ int classify_row(const SampleParams& p, int64_t row, int& K) {
  K = p.top_k[row];
  if (K <= 0 || (int64_t)K >= p.vocab) K = (int)p.vocab;
  if (p.temperature[row] < kSamplingEps) return (int)kGreedy;
  return K <= kFastK ? (int)kFast : (int)kGeneral;
}

}  // namespace tlx
#include "sampler_wide.cuh"
#include "sampler_stream.cuh"
#include "sampler_rows.cuh"
namespace tlx {

// ---- the kernels --------------------------------------------------------------------------
constexpr size_t kSlicesSmem = kSharedHeader + kUnionBytes + 2 * (size_t)kSliceBytes + sizeof(Control);
constexpr size_t kMergeSmem = kSharedHeader + kUnionBytes;

// Kernel 1: persistent CTAs stream the slices (statically assigned: CTA c takes the items
// c, c + grid, ...) and write one record per slice.  Nothing in the per-slice path waits on
// a global-memory round trip: while the memory system is saturated by the bulk copies such a
// round trip costs several microseconds, more than a slice's whole share of the time.
template <int DT>
__global__ void __launch_bounds__(kThreads, 2) sample_slices_kernel(SampleParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  unsigned char* uni = smem_raw + kSharedHeader;
  unsigned char* slice_base = uni + kUnionBytes;
  Control& ctl = *reinterpret_cast<Control*>(uni + kUnionBytes + 2 * (size_t)kSliceBytes);
  uint32_t* win = reinterpret_cast<uint32_t*>(uni);
  constexpr int kPublisher = kThreads - 1;

  const Geometry g{p.S, p.chunk_elems, p.nchunks, p.vocab, 31 - __clz(p.chunk_elems), p.div_magic};
  const int total = (int)(p.rows * p.S);

  if (threadIdx.x == 0) {
    mbar_init(&ctl.mbar[0], 1);
    mbar_init(&ctl.mbar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl.timeout = 0;
  }
  __syncthreads();
  auto load = [&](int item, int b) {
    if (item < total && warp_id() == 0) {
      const int rp = g.div_S(item);
      issue_slice_load<DT>(p, g, rp, item - rp * p.S, slice_base + (size_t)b * kSliceBytes, &ctl.mbar[b]);
    }
  };
  // Row parameters are fetched one slice ahead, so that the per-slice path never waits for them:
  // packed as top-k in the low bits, bit 30 = greedy, bit 31 = general.
  auto fetch_class = [&](int item) -> uint32_t {
    if (item >= total) return 0u;
    int K;
    const int cls = classify_row(p, g.div_S(item), K);
    return cls == kGreedy ? (1u << 30)
           : cls == kGeneral ? ((1u << 31) | ((int64_t)K >= p.vocab ? (1u << 29) : 0u))
                             : (uint32_t)K;
  };

  // Work list.  Small batches of general rows (only_general): every CTA first compacts the wanted
  // rows into shared memory (each thread classifies a few rows, one block scan), so that the
  // items (wanted row, slice) can be dealt out evenly: CTA c takes the items c, c + grid, ...
  // Otherwise the items are simply (row, slice) = (i / S, i % S) over all rows.
  constexpr int kPlanRows = 4 * kThreads;
  static_assert(kPlanRows <= 1024, "rows_list holds 1024 rows");
  const bool compact = p.only_general && p.rows <= kPlanRows;
  int n_items = total;
  if (compact) {
    uint32_t flags = 0, cnt = 0;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int r = threadIdx.x * 4 + h;
      if (r < p.rows) {
        const uint32_t packed = fetch_class(r * p.S);
        if ((packed >> 31) && (!p.final_pass || ((packed >> 29) & 1u))) { flags |= 1u << h; ++cnt; }
      }
    }
    uint32_t tot;
    uint32_t pos = block_scan_incl<uint32_t>(cnt, s.scan_u32, &tot, ShflUpU32()) - cnt;
    unsigned short* rows_list = ctl.rows_list;
#pragma unroll
    for (int h = 0; h < 4; ++h)
      if (flags & (1u << h)) rows_list[pos++] = (unsigned short)(threadIdx.x * 4 + h);
    n_items = (int)tot * p.S;
    __syncthreads();
  }
  const int stride = gridDim.x;
  const int n_my = (int)blockIdx.x < n_items ? (n_items - 1 - (int)blockIdx.x) / stride + 1 : 0;
  uint32_t phases = 0;   // bit i: parity to wait for on barrier i
  for (int base = 0; base < n_my; base += 64) {
    if (threadIdx.x == 0) ctl.list_n = 0;
    __syncthreads();
    if (threadIdx.x < 64 && base + (int)threadIdx.x < n_my) {
      int item = blockIdx.x + (base + threadIdx.x) * stride;
      if (compact) {   // (wanted row index, slice) -> (row, slice)
        const int wi = g.div_S(item);
        item = (int)ctl.rows_list[wi] * p.S + (item - wi * p.S);
      }
      const uint32_t packed = fetch_class(item);
      // general rows only when asked; the final pass further wants the top-k filter to be disabled
      if ((!p.only_general || (packed >> 31)) && (!p.final_pass || ((packed >> 29) & 1u))) {
        const int pos = atomicAdd(&ctl.list_n, 1);
        ctl.list[pos] = item;
        ctl.list_cls[pos] = packed;
      }
    }
    __syncthreads();
    const int nl = ctl.list_n;
    if (nl > 0) load(ctl.list[0], 0);
    if (nl > 1) load(ctl.list[1], 1);
    // One block-wide barrier per slice in the common case: warps reduce their share of the slice
    // on their own, then meet once; after that warp 0 refills the buffer and the last thread
    // writes the record's header while everybody else already waits for the next slice.
    for (int j = 0; j < nl; ++j) {
      const int b = j & 1;
      unsigned char* buf = slice_base + (size_t)b * kSliceBytes;
      const int cur = ctl.list[j];
      const uint32_t cls_cur = ctl.list_cls[j];
      if (!mbar_wait(&ctl.mbar[b], (phases >> b) & 1u)) ctl.timeout = 1;
      phases ^= 1u << b;

      const int64_t row = g.div_S(cur);
      const int sl = cur - (int)row * p.S;
      const int elems = g.slice_elems(sl);
      const int cls = (cls_cur >> 30) & 1u ? (int)kGreedy : (cls_cur >> 31) ? (int)kGeneral : (int)kFast;
      const int K = (int)(cls_cur & 0x1FFFFFFFu);
      WarpResults& wr = ctl.wr[b];
      if (p.final_pass) {
        if constexpr (DT == TLX_BF16) reduce_slice_final_bf16(p, g, row, sl, buf, elems, s, uni);
      } else if (cls == kGreedy) {
        reduce_slice_greedy<DT>(buf, elems, wr);
      } else if (cls == kFast) {
        uint64_t* segment = reinterpret_cast<uint64_t*>(record_payload(p, row, sl)) + warp_id() * kWarpCap;
        reduce_slice_fast<DT>(g, sl, K, buf, elems, segment,
                              reinterpret_cast<unsigned short*>(uni) + warp_id() * kWarpHits, wr);
      } else if constexpr (DT == TLX_BF16) {
        reduce_slice_general_bf16(p, g, row, sl, buf, elems, s, win);
      }
      __syncthreads();   // the slice is reduced and its buffer is free
      if (j + 2 < nl) load(ctl.list[j + 2], b);
      if (p.final_pass) {
        // count the slice on its row; whoever delivers the last one turns the row's best into its token
        if (threadIdx.x == kPublisher) {
          RowState* rs = p.rowstate + row;
          __threadfence();
          if (atomicAdd(&rs->done, 1) == p.S - 1) {
            __threadfence();
            const unsigned long long best = atomicMax(&rs->best, 0ull);
            p.out_tokens[row] = 0x7FFFFFFF - (int32_t)(uint32_t)best;
          }
        }
      } else if (threadIdx.x == kPublisher) {
        SliceHeader* hdr = record_header(p, row, sl);
        if (cls == kGreedy) {
          unsigned long long best = 0;
          for (int w = 0; w < kWarps; ++w) best = wr.top[w] > best ? wr.top[w] : best;
          const int q = 0x7FFFFFFF - (int)(uint32_t)best;
          const int64_t col = elems > 0 ? g.column(sl, q) : 0;
          hdr->top = (best & 0xFFFFFFFF00000000ull) | (uint32_t)(0x7FFFFFFF - (int32_t)col);
        } else if (cls == kFast) {
          int over = 0;
          for (int w = 0; w < kWarps; ++w) { hdr->wcount[w] = wr.count[w]; over |= wr.overflow[w]; }
          hdr->cutoff_bin = wr.cutoff_bin;
          hdr->overflow = over;
        }
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0 && ctl.timeout) atomicOr(&p.counters[1], 1);
}


// Kernel 2: one CTA per row turns the row's slice records into a token.
template <int DT>
__global__ void __launch_bounds__(kRowThreads) sample_merge_kernel(SampleParams p) {
  using T = typename Elem<DT>::type;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  unsigned char* uni = smem_raw + kSharedHeader;
  uint64_t* cand = reinterpret_cast<uint64_t*>(uni);
  uint32_t* win = reinterpret_cast<uint32_t*>(uni);
  double* massbins = reinterpret_cast<double*>(uni);
  const int64_t row = blockIdx.x;
  int K;
  const int cls = classify_row(p, row, K);
  const float pp = p.top_p[row], T_ = p.temperature[row];
  int status = cls == kGeneral ? kStatusGeneral : 0;
  int tok;
  if (cls == kGreedy) tok = merge_row_greedy(p, row, s);
  else if (cls == kFast) tok = merge_row_fast<DT>(p, row, K, pp, T_, s, cand, &status);
  else if constexpr (DT == TLX_BF16) tok = merge_row_general_bf16(p, row, K, pp, T_, s, win);
  else tok = general_row_radix<DT>(reinterpret_cast<const T*>(p.logits) + row * p.row_stride, p.vocab, K, pp, T_,
                                   p.noise, row + p.dim0_offset, s, massbins);
  if (threadIdx.x == 0) {
    if (p.counters[1]) status |= kStatusTimeout;
    p.out_tokens[row] = tok;
    if (p.out_status) p.out_status[row] = status;
  }
}

// ---- one CTA per row ---------------------------------------------------------------------------
// For batches of at least one row per CTA slot the row is not cut up: a CTA streams its row
// through the two slice buffers tile by tile (one contiguous bulk copy each) and keeps the
// selection state of collect_row in shared memory across the tiles -- a 4096-bin histogram of
// what was collected, the candidate list, and the threshold bin, which rises as soon as the
// histogram shows K collected elements at or above a higher bin.  After the first tile the
// per-tile work is one packed compare per two elements; everything (candidates, tail, token)
// stays inside the CTA, so there is no workspace traffic and no second kernel.
// Rows without any filter: per element the screened score x / T + gumbel(u), the thread's two best.
struct PlainScore {
  float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
  uint32_t k1 = 0;
  int c1 = 0x7FFFFFFF;
  __device__ __forceinline__ void offer(float x, float u, int col, float inv_T) {
    const float a = x * inv_T + gumbel_screen(u);
    if (a > a1) { a2 = a1; a1 = a; k1 = f32_key(x); u1 = u; c1 = col; }
    else if (a > a2) a2 = a;
  }
};

// One tile of such a row: the noise of a vector's columns is contiguous (a vector never straddles
// two chunks), so it comes in with 16-byte loads, two vectors of the thread at a time.
template <int DT>
__device__ __forceinline__ void score_tile_plain(const SampleParams& p, const Geometry& g, int t, int64_t nrow,
                                                 const unsigned char* buf, int elems, float inv_T, PlainScore& sc) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int kPair = 2;
  const int nvec = elems / VEC;
  const uint4* vp = reinterpret_cast<const uint4*>(buf);
  const bool noise_vec = p.noise.dense && ((reinterpret_cast<uintptr_t>(p.noise.dense) & 15) == 0) &&
                         ((p.noise.stride & 3) == 0);
  const float* nbase = p.noise.dense ? p.noise.dense_row(nrow) : nullptr;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += kPair * (int)blockDim.x) {
    uint4 v[kPair];
    float4 nz[kPair][VEC / 4];
    int col0[kPair];
#pragma unroll
    for (int u = 0; u < kPair; ++u) {
      const int i = i0 + u * (int)blockDim.x;
      col0[u] = -1;
      if (i < nvec) {
        v[u] = vp[i];
        col0[u] = (int)g.column(t, i * VEC);
        if (noise_vec) {
#pragma unroll
          for (int q = 0; q < VEC / 4; ++q) nz[u][q] = __ldg(reinterpret_cast<const float4*>(nbase + col0[u]) + q);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kPair; ++u) {
      if (col0[u] < 0) continue;
      T e[VEC];
      memcpy(e, &v[u], sizeof(uint4));
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        float un;
        if (noise_vec) {
          const float4 f = nz[u][j >> 2];
          un = (j & 3) == 0 ? f.x : (j & 3) == 1 ? f.y : (j & 3) == 2 ? f.z : f.w;
        } else {
          un = p.noise.at(nrow, (int64_t)col0[u] + j);
        }
        sc.offer(elem_as_float<DT>(e[j]), un, col0[u] + j, inv_T);
      }
    }
  }
  for (int q = nvec * VEC + threadIdx.x; q < elems; q += blockDim.x) {   // ragged end of the row's last tile
    const int col = (int)g.column(t, q);
    sc.offer(elem_as_float<DT>(slice_elem<DT>(buf, q)), p.noise.at(nrow, col), col, inv_T);
  }
}

constexpr size_t kRowsSmem = kSharedHeader + kUnionBytes + 2 * (size_t)kSliceBytes + sizeof(Control);

template <int DT>
__global__ void __launch_bounds__(kRowsKThreads, 2) sample_rows_kernel(SampleParams p) {
  using T = typename Elem<DT>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  unsigned char* uni = smem_raw + kSharedHeader;
  unsigned char* slice_base = uni + kUnionBytes;
  Control& ctl = *reinterpret_cast<Control*>(uni + kUnionBytes + 2 * (size_t)kSliceBytes);
  uint64_t* cand = reinterpret_cast<uint64_t*>(uni);
  uint32_t* win = reinterpret_cast<uint32_t*>(uni);
  double* massbins = reinterpret_cast<double*>(uni);
  // while a row is collected its histogram area is idle and holds the warps' hit lists
  unsigned short* hits = reinterpret_cast<unsigned short*>(s.hist) + warp_id() * (kHistBins * 2 / kRowWarps);

  // The tiles of a row are its S interleaved slices: every tile is a sample of the whole row,
  // so the threshold estimated on the first one is already right for the others.
  const Geometry g{p.S, p.chunk_elems, p.nchunks, p.vocab, 31 - __clz(p.chunk_elems), p.div_magic};
  const int64_t n = p.vocab;
  if (threadIdx.x == 0) {
    mbar_init(&ctl.mbar[0], 1);
    mbar_init(&ctl.mbar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl.timeout = 0;
  }
  __syncthreads();
  uint32_t phases = 0;

  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* rowp = reinterpret_cast<const T*>(p.logits) + row * p.row_stride;
    auto load = [&](int t, int b) {
      if (t < p.S && warp_id() == 0)
        issue_slice_load<DT>(p, g, row, t, slice_base + (size_t)b * kSliceBytes, &ctl.mbar[b]);
    };
    int K;
    const int cls = classify_row(p, row, K);
    const float pp = p.top_p[row], T_ = p.temperature[row];
    int status = 0, tok = 0;
    // rows without top-k only get their threshold here: the final pass is the third kernel's
    // No filter at all (top-k disabled, top_p >= 1): a plain Gumbel arg-max over the row, streamed here.
    const bool plain = cls == kGeneral && (int64_t)K >= n && pp >= 1.0f && !p.have_records;
    if (DT == TLX_BF16 && p.wide_elsewhere && cls == kGeneral && (int64_t)K >= n && !plain) continue;   // the cluster kernel's
    const bool deferred = DT == TLX_BF16 && cls == kGeneral && (int64_t)K >= n && p.have_records;
    if (!deferred) {
      load(0, 0);
      load(1, 1);
    }

    if (plain) {
      status = kStatusGeneral;
      const int64_t nrow = row + p.dim0_offset;
      PlainScore sc;
      for (int t = 0; t < p.S; ++t) {
        const int b = t & 1;
        if (!mbar_wait(&ctl.mbar[b], (phases >> b) & 1u)) ctl.timeout = 1;
        phases ^= 1u << b;
        score_tile_plain<DT>(p, g, t, nrow, slice_base + (size_t)b * kSliceBytes, g.slice_elems(t), 1.0f / T_, sc);
        __syncthreads();   // the tile is consumed, its buffer is free
        load(t + 2, b);
      }
      // the best screened score and what lies within the slack below it (see tail_bf16_hist)
      const Best top = block_best(Best{sc.a1, sc.c1}, s);
      const float cut = top.y - (kGumbelSlack + 1e-5f * fabsf(top.y));
      const int leaders = __syncthreads_count(sc.a1 >= cut);
      const int crowded = __syncthreads_or(sc.a2 >= cut);
      if (crowded || top.tok == 0x7FFFFFFF) {
        tok = final_argmax<DT>(rowp, n, T_, 0u, false, 0u, 0u, false, p.noise, nrow, s);   // rare: whole-row routine
      } else if (leaders == 1) {
        tok = top.tok;
      } else {
        Best best{-INFINITY, 0x7FFFFFFF};
        if (sc.a1 >= cut) best = Best{__fdiv_rn(key_f32(sc.k1), T_) + gumbel_exact(sc.u1), sc.c1};
        tok = block_best(best, s).tok;
      }
    } else if (cls == kGeneral) {
      status = kStatusGeneral;
      bool done = false;
      if constexpr (DT == TLX_BF16) {
        if (deferred) {
          // The slices kernel left this row's histograms in the workspace; they give the top-p
          // threshold, which goes to the row's state for the final pass.
          const int vstar16 = merge_row_general_bf16(p, row, K, pp, T_, s, win, true);
          if (threadIdx.x == 0) {
            RowState* rs = p.rowstate + row;
            rs->min_key = vstar16 == 0 ? 0u : key16_to_key32((uint32_t)vstar16);
            rs->thr = vstar16 == 0 ? -INFINITY : key16_value(vstar16);
            rs->best = 0ull;
            rs->done = 0;
            if (p.out_status) p.out_status[row] = status;
          }
          __syncthreads();
          continue;
        }
      }
      if (!done) {
        // drain the two copies that are in flight, then take the whole-row path from global memory
        for (int t = 0; t < 2 && t < p.S; ++t) {
          if (!mbar_wait(&ctl.mbar[t], (phases >> t) & 1u)) ctl.timeout = 1;
          phases ^= 1u << t;
        }
        __syncthreads();
        if constexpr (DT == TLX_BF16) {
          RowPreset pre;
          tok = general_row_bf16<kWin>(rowp, n, K, pp, T_, p.noise, row + p.dim0_offset, s, win, pre);
        } else {
          tok = general_row_radix<DT>(rowp, n, K, pp, T_, p.noise, row + p.dim0_offset, s, massbins);
        }
      }
    } else {
      unsigned long long wbest = 0;   // greedy: this warp's running arg-max (key << 32 | 0x7FFFFFFF - column)
      // A first threshold that turns out too high (fewer than K candidates at the end of the row)
      // costs one more pass over the row with a lower one, then a second, then the exact select.
      int forced_bin = -1;
      uint32_t fine_key = 0u;   // first threshold at 16-bit granularity (at or above the lower edge of bin s.bin)
      for (int attempt = 0;; ++attempt) {
      if (threadIdx.x == 0) { s.fill = 0; s.bin = 0; s.above = 0; s.refinements = 0; }
      __syncthreads();
      for (int t = 0; t < p.S; ++t) {
        const int b = t & 1;
        unsigned char* buf = slice_base + (size_t)b * kSliceBytes;
        const int elems = g.slice_elems(t);
        if (!mbar_wait(&ctl.mbar[b], (phases >> b) & 1u)) ctl.timeout = 1;
        phases ^= 1u << b;
        if (cls == kGreedy) {
          reduce_slice_greedy<DT>(buf, elems, ctl.wr[b]);
          if (lane_id() == 0) {
            const unsigned long long v = ctl.wr[b].top[warp_id()];
            if (v) {
              const int64_t col = g.column(t, 0x7FFFFFFF - (int)(uint32_t)v);
              const unsigned long long c = (v & 0xFFFFFFFF00000000ull) | (uint32_t)(0x7FFFFFFF - (int32_t)col);
              wbest = c > wbest ? c : wbest;
            }
          }
        } else {
          if (t == 0 && forced_bin >= 0) {
            if (threadIdx.x == 0) s.bin = forced_bin;
            fine_key = 0u;
            __syncthreads();
          } else if (t == 0) {
            // First threshold, from the maxima of the threads' elements: aim at 1.25 K + 48 elements of
            // the ROW, i.e. that fraction of this tile, at the granularity of 16-bit keys (a whole bin
            // more than needed can double the candidates).  Too high an estimate is caught at the end
            // (fewer than K candidates), too low a one by the refinement below.
            const int nvec = elems / VEC;
            const float frac = fminf(1.f, (1.25f * (float)K + 48.f) / (float)n);
            const int vec_per_thread = (nvec + (int)blockDim.x - 1) / (int)blockDim.x;
            int vecs = (int)(0.7f / (frac * VEC) + 0.5f);
            vecs = vecs < 1 ? 1 : (vecs > vec_per_thread ? vec_per_thread : vecs);
            const uint32_t tkey = thread_max_key<DT>(buf, nvec, vecs);
            const int my_key16 = ((int)threadIdx.x < nvec) ? (int)(tkey >> 16) : -1;
            const int holders = nvec < (int)blockDim.x ? nvec : (int)blockDim.x;
            // two and a half standard deviations of the count of holders above the wanted threshold as margin
            float wantf = (float)holders * (1.f - __expf(-(float)(vecs * VEC) * frac));
            wantf += 2.5f * sqrtf(wantf);
            int want = (int)(wantf + 0.999f);
            want = want < 1 ? 1 : (want > holders ? holders : want);
            const int k16 = (frac >= 0.5f || nvec == 0) ? 0 : vote_threshold_key16(my_key16, want);
            fine_key = (uint32_t)k16 << 16;
            if (threadIdx.x == 0) s.bin = k16 >> 4;
            __syncthreads();
          }
          const uint32_t bin_key = (uint32_t)s.bin << kHistShift;   // the bin only moves inside the refinement
          collect_tile<DT, kRowWarps>(buf, elems, bin_key > fine_key ? bin_key : fine_key, s, cand, hits,
                                      [&](int q) { return g.column(t, q); });
        }
        // The tile is consumed, its buffer is free.  The same barrier carries the decision to raise the
        // threshold, which is due when the candidate list fills up (and once at the end for the sorting
        // tail, which wants few candidates).  It must be the same for every thread (the refinement has
        // barriers of its own), but a thread that read the fill level after the barrier could see what
        // a faster warp has already appended from the next tile: so every thread reads it before, and
        // the block takes the OR.
        const int fill_seen = s.fill;
        // (half the list for the usual top_k; a large top_k fills more than that by itself and waits longer)
        const int refine_at = 2 * K > kMergeCap / 2 ? (2 * K < kMergeCap - 512 ? 2 * K : kMergeCap - 512) : kMergeCap / 2;
        const int refine_now = __syncthreads_or(
            cls == kFast && (fill_seen > refine_at || (t == p.S - 1 && DT != TLX_BF16 && fill_seen > 2 * K + 64)));
        load(t + 2, b);
        if (refine_now) {
          __syncthreads();   // nobody is ahead in the next tile while the fill level is looked at again
          if (s.fill <= kMergeCap) refine_candidates(s, cand, K);
        }
      }
      if (cls == kGreedy) break;
      const int m_try = s.fill, bin_try = s.bin;
      __syncthreads();
      if (m_try >= K || bin_try == 0 || attempt == 2) break;
      forced_bin = bin_try - (attempt == 0 ? 1 : 4);
      forced_bin = forced_bin < 0 ? 0 : forced_bin;
      status |= kStatusRedone;
      load(0, 0);
      load(1, 1);
      }
      if (cls == kGreedy) {
        unsigned long long* slot = reinterpret_cast<unsigned long long*>(s.scan_f64);
        if (lane_id() == 0) slot[warp_id()] = wbest;
        __syncthreads();
        unsigned long long best = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = slot[w] > best ? slot[w] : best;
        tok = 0x7FFFFFFF - (int32_t)(uint32_t)best;
        __syncthreads();
      } else {
        int m = s.fill;
        __syncthreads();
        if (m > kMergeCap || m < K) {   // overflow (huge tie groups) or an estimate that was too high: exact select
          exact_select_row<DT>(rowp, n, K, s, cand);
          m = K;
          status |= kStatusRedone;
          __syncthreads();
        }
        tok = -1;
        if constexpr (DT == TLX_BF16) if (tok < 0) tok = tail_bf16_hist(p, row, K, pp, T_, m, s, cand);
        if (tok < 0) {
          __syncthreads();
          sort_candidates(cand, m);
          const int64_t nrow = row + p.dim0_offset;
          tok = sample_tail<4>(
              K, pp, T_, s, [&](int i) { return key_f32(cand_key(cand[i])); },
              [&](int i) { return (int)cand_low(cand[i]); },
              [&](int i) { return p.noise.at(nrow, (int64_t)cand_low(cand[i])); });
        }
      }
    }
    if (threadIdx.x == 0) {
      if (ctl.timeout) status |= kStatusTimeout;
      p.out_tokens[row] = tok;
      if (p.out_status) p.out_status[row] = status;
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

struct MergeParams {
  const float* cand_vals;
  const int32_t* cand_idx;
  const float* cand_noise;
  int n_cand, k_per_block;
  int64_t block_stride, row_stride;
  const int32_t* top_k;
  const float* top_p;
  const float* temperature;
  int32_t* out;
  // exchange mode (xbuf non-null): the candidates are read from this rank's exchange buffer, set by set
  unsigned char* xbuf;
  size_t off_flags[2], off_cand[2];
  int world;
  int64_t rows;
  int32_t* status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Number of entries of the ascending list blk[0..len) whose high word is smaller than `target`.  The high
// word is the inverted key; it never reaches 0xFFFFFFFF (no key is 0), so target may be a high word plus one.
__device__ __forceinline__ int count_high_below(const uint64_t* blk, int len, uint32_t target) {
  const uint32_t* hi = reinterpret_cast<const uint32_t*>(blk) + 1;
  int lo = 0;
  while (len > 0) {
    const int half = len >> 1;
    if (hi[2 * (lo + half)] < target) { lo += half + 1; len -= half + 1; }
    else len = half;
  }
  return lo;
}

// One CTA per row.  The shards' blocks arrive sorted (value desc, token asc), which the kernel checks: a
// candidate's place in the merged order is then its place in its own block plus, for every other block,
// the number of entries that precede it there (a binary search), and only places below K are filled; one
// comparison per block rules most candidates out before any search.
// Unsorted blocks take the bitonic network over all candidates instead.
__global__ void __launch_bounds__(kMergeThreads) merge_and_sample_kernel(MergeParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + ((sizeof(SelectShared) + 15) & ~size_t(15)));
  const int n_cand = p.n_cand, kpb = p.k_per_block;
  int P = 2;
  while (P < n_cand) P <<= 1;
  uint64_t* merged = cand + P;
  const int64_t r = blockIdx.x;

  const float* v = p.cand_vals;
  const int32_t* id = p.cand_idx;
  const float* un = p.cand_noise;
  ExchangeHeader* xh = reinterpret_cast<ExchangeHeader*>(p.xbuf);
  uint32_t* flag = nullptr;
  if (xh) {
    const uint32_t par = *reinterpret_cast<volatile const uint32_t*>(&xh->step) & 1u;
    const size_t plane = (size_t)p.rows * kpb;
    v = reinterpret_cast<const float*>(p.xbuf + p.off_cand[par]);
    id = reinterpret_cast<const int32_t*>(v) + plane;
    un = v + 2 * plane;
    flag = reinterpret_cast<uint32_t*>(p.xbuf + p.off_flags[par]) + r;
    // a call whose extents are not the buffer's reads nothing: token -1, status 2
    if (xh->rows != (uint32_t)p.rows || xh->k_cand != (uint32_t)kpb || xh->world != (uint32_t)p.world) {
      if (threadIdx.x == 0) {
        atomicExch(&xh->error, 2u);
        if (p.status) atomicExch(p.status, 2);
        p.out[r] = -1;
      }
      return;
    }
    if (threadIdx.x == 0) {
      // every rank's block of this row has arrived when the word reads `world`; two seconds at most
      const unsigned long long t0 = global_timer_ns();
      bool ok = false;
      for (int it = 0; it < (1 << 24); ++it) {
        if (ld_acquire_sys_u32(flag) >= (uint32_t)p.world) { ok = true; break; }
        if (global_timer_ns() - t0 > 2000000000ull) break;
        __nanosleep(100);
      }
      if (!ok) {
        atomicExch(&xh->error, 1u);
        if (p.status) atomicExch(p.status, 1);
      }
    }
    __syncthreads();
  }
  v += r * p.row_stride;
  id += r * p.row_stride;
  un += r * p.row_stride;
  // block of candidate i without an integer division: (i + 0.5) / kpb is at least 0.5 / kpb away from an
  // integer and i < 8192, far more than the product's rounding error
  const float inv_kpb = 1.0f / (float)kpb;
  auto block_of = [&](uint32_t i) { return (int)(((float)i + 0.5f) * inv_kpb); };
  auto at = [&](uint32_t i) {
    const int b = block_of(i);
    return (int64_t)b * p.block_stride + (int64_t)((int)i - b * kpb);
  };
  // low word = position in the gathered list: shards are laid side by side in ascending
  // token order, so position order equals token order among equal values
  int unsorted = 0;
  for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
    const float x = xh ? __ldcg(v + at(i)) : v[at(i)];
    cand[i] = cand_make(f32_key(x), (uint32_t)i);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_cand; i += blockDim.x)
    if (i != block_of(i) * kpb && cand[i - 1] > cand[i]) unsorted = 1;
  unsorted = __syncthreads_or(unsorted);
  int K = p.top_k[r];
  if (K <= 0 || K > n_cand) K = n_cand;
  const uint64_t* top = cand;
  if (unsorted) {
    sort_candidates(cand, n_cand);
  } else if (n_cand > kpb) {
    // Step 1, every candidate: q entries of its own block precede it; if entry K-1-q of another block does
    // too, so do that block's first K-q entries and its place is K or more.  The others (K and a few more
    // per block) are listed.  Step 2, one listed candidate per thread: a binary search per other block.
    const int blocks = n_cand / kpb;
    uint32_t* listed = reinterpret_cast<uint32_t*>(merged + n_cand);
    if (threadIdx.x == 0) s.fill = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
      const int b = block_of(i);
      const int q = i - b * kpb;
      if (q >= K) continue;
      const uint64_t c = cand[i];
      const int probe = K - 1 - q;
      bool out = false;
      if (probe < kpb)
        for (int o = 0; o < blocks && !out; ++o) out = o != b && cand[o * kpb + probe] < c;
      if (!out) {
        // the same with the places shared out evenly: if entry d-1 of EVERY other block precedes it, with
        // d * (blocks - 1) >= K - q, its place is K or more as well
        const int d = (K - q + blocks - 2) / (blocks - 1);
        if (d - 1 < kpb) {
          bool all = true;
          for (int o = 0; o < blocks && all; ++o) all = o == b || cand[o * kpb + d - 1] < c;
          out = all;
        }
      }
      if (!out) listed[atomicAdd(&s.fill, 1)] = (uint32_t)i;
    }
    __syncthreads();
    const int nlisted = s.fill;
    for (int l = threadIdx.x; l < nlisted; l += blockDim.x) {
      const int i = (int)listed[l];
      const int b = block_of(i);
      const int q = i - b * kpb;
      const uint64_t c = cand[i];
      int place = q;
      const int span = min(kpb, K - q);   // a block's entries from `span` on cannot change the verdict
      // entries of another block that precede c: a smaller high word (the inverted key), or an equal one in a
      // block before c's own (positions, the low words, grow with the block) -- a search on the high words
      const uint32_t chi = (uint32_t)(c >> 32);
      for (int o = 0; o < blocks && place < K; ++o)
        if (o != b) place += count_high_below(cand + o * kpb, span, chi + (o < b ? 1u : 0u));
      if (place < K) merged[place] = c;
    }
    __syncthreads();
    top = merged;
  }
  const float T_ = p.temperature[r];
  int tok;
  if (T_ < kSamplingEps) {
    tok = id[at(cand_low(top[0]))];
  } else {
    tok = sample_tail<2>(
        K, p.top_p[r], T_, s, [&](int i) { return key_f32(cand_key(top[i])); },
        [&](int i) { return (int)id[at(cand_low(top[i]))]; }, [&](int i) { return un[at(cand_low(top[i]))]; });
  }
  if (threadIdx.x == 0) {
    p.out[r] = tok;
    if (xh) {
      // the row is consumed: clear its arrival word; the last row's CTA of the step advances the step
      *reinterpret_cast<volatile uint32_t*>(flag) = 0u;
      __threadfence();
      if (atomicAdd(&xh->done, 1u) == gridDim.x - 1) {
        *reinterpret_cast<volatile uint32_t*>(&xh->done) = 0u;
        __threadfence();
        atomicAdd(&xh->step, 1u);
      }
    }
  }
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
                                                            int64_t cols, uint32_t k0, uint32_t k1,
                                                            const uint32_t* __restrict__ key_dev, int64_t dim1,
                                                            int axis, int32_t* __restrict__ out) {
  __shared__ float sy[8];
  __shared__ int sp[8];
  if (key_dev) { k0 = __ldg(key_dev); k1 = __ldg(key_dev + 1); }
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
    const float a = l + gumbel_screen(u);
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

// A helper stream with the two events that fork it from and join it to the caller's stream.
// One per host thread and device, made on first use and kept for the life of the process.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
// Off unless tlx_init asked for it: a library call then creates no CUDA object of its own, which a
// caller inside a stream capture or under a tracing compiler relies on.
static std::atomic<int> g_side_stream_enabled{0};
static SideStream* side_stream(bool create_only = false) {
  static thread_local SideStream cache[64];
  if (!g_side_stream_enabled.load(std::memory_order_relaxed) && !create_only) return nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  SideStream& ss = cache[dev];
  if (!ss.stream) {
    cudaStream_t st = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;   // the caller falls back to its own stream
    }
    ss.stream = st; ss.fork = a; ss.join = b;
  }
  return &ss;
}

static int device_sm_count() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

struct SliceLayout {
  int S, chunk_elems, nchunks;
};
static SliceLayout slice_layout(int64_t vocab, int elem_bytes) {
  SliceLayout l;
  l.chunk_elems = kChunkBytes / elem_bytes;
  l.nchunks = (int)((vocab + l.chunk_elems - 1) / l.chunk_elems);
  l.S = (l.nchunks + kChunksPerSlice - 1) / kChunksPerSlice;
  return l;
}
// workspace: [flags | one RowState per row | one record per (row, slice)]
static size_t counters_bytes(int64_t rows) { return 256 + (((size_t)rows * sizeof(RowState) + 255) & ~size_t(255)); }


// ---- streaming path (sampler_stream.cuh): workspace layout and launches ---------------------------
struct StreamLayout {
  int P, part_chunks, nchunks, nfin;
  size_t off_desc, off_counts, off_lump, off_wbest, off_flag, off_rowdone, off_state, off_records, off_hist, off_cands, off_timeline = 0, bytes;
};
static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
static StreamLayout stream_layout(int64_t rows, int64_t vocab) {
  StreamLayout l;
  l.nchunks = (int)((vocab * 2 + kStChunk - 1) / kStChunk);
  l.part_chunks = (l.nchunks + kStMaxParts - 1) / kStMaxParts;
  if (l.part_chunks < 2) l.part_chunks = 2;
  l.P = (l.nchunks + l.part_chunks - 1) / l.part_chunks;
  l.nfin = (int)((vocab * 2 + kFinChunk - 1) / kFinChunk);
  size_t o = 256;   // [0]: error flag, [1]: item counter
  l.off_desc = o;    o = align256(o + (size_t)rows * sizeof(StreamDesc));
  l.off_counts = o;  o = align256(o + (size_t)rows * l.P * kStWarps * sizeof(int));
  l.off_lump = o;    o = align256(o + (size_t)rows * l.P * sizeof(double));
  l.off_wbest = o;   o = align256(o + (size_t)rows * sizeof(unsigned long long));
  l.off_flag = o;    o = align256(o + (size_t)rows * sizeof(int));
  l.off_rowdone = o; o = align256(o + (size_t)rows * sizeof(int));
  l.off_state = o;   o = align256(o + (size_t)rows * sizeof(WideState));
  l.off_records = o; o = align256(o + (size_t)rows * l.nfin * sizeof(FinRecord));
  l.off_hist = o;    o = align256(o + (size_t)rows * kStWin * sizeof(uint32_t));
  l.off_cands = o;   o = align256(o + (size_t)rows * l.P * kStWarps * kStWarpCap * sizeof(uint32_t));
#ifdef TLX_TIMELINE
  l.off_timeline = o; o = align256(o + (size_t)4 * 8192 * 16 * sizeof(long long));
#endif
  l.bytes = o;
  return l;
}
// bf16 rows that bulk copies can address, long enough for the prologue's sample, few enough for the
// kernels' per-row tables in shared memory, short enough for 16 parts of at most ten chunks
static bool stream_path_serves(int dtype, int64_t rows, int64_t vocab, int64_t row_stride, const void* logits) {
  if (dtype != TLX_BF16 || vocab < kStMinVocab || rows > kStMaxRows) return false;
  if ((reinterpret_cast<uintptr_t>(logits) & 15) != 0 || ((row_stride * 2) & 15) != 0 || ((vocab * 2) & 15) != 0) return false;
  return stream_layout(rows, vocab).part_chunks <= kStMaxPartChunks;
}

// Diagnostic switch for timing the stages of the streaming path one by one (environment variable
// TLX_SAMPLE_STAGES = 1..3: launch only the first n kernels; +16: the stream kernel only takes the
// chunks, the streaming floor; +32 / +64: the final pass without its scoring / without its records).
// Unset in normal use: all three kernels run.
static int debug_stages() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("TLX_SAMPLE_STAGES");
    v = e ? atoi(e) : 3;
    if (v <= 0) v = 3;
  }
  return v;
}

// Launches a kernel that may start while its predecessor on the stream still runs (programmatic dependent
// launch): the kernel does whatever needs none of the predecessor's results and then executes
// griddepcontrol.wait, which returns when the predecessor has finished and its writes are visible.  Where
// the attribute is not accepted the kernel is launched in plain stream order (the wait is then a no-op).
template <typename... Params, typename... Args>
static int launch_dependent(void (*kernel)(Params...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                            const char* what, Args... args) {
  static bool programmatic = getenv("TLX_NO_DEPENDENT_LAUNCH") == nullptr;
  if (programmatic) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...) == cudaSuccess) {
      count_launch();
      return TLX_OK;
    }
    cudaGetLastError();
    programmatic = false;
  }
  kernel<<<grid, block, smem, st>>>(static_cast<Params>(args)...);
  TLX_CHECK_LAUNCH(what);
  return TLX_OK;
}

// Row-per-CTA path (sampler_rows.cuh): no workspace; two CTAs per SM, more rows than that are taken in turn.
static int launch_rows_path(cudaStream_t st, const SampleParams& sp) {
  const int sms = device_sm_count();
  RowsParams p{};
  p.sp = sp;
  p.nchunks = (int)((sp.vocab * 2 + kRwChunk - 1) / kRwChunk);
  p.row_bytes = sp.vocab * 2;
  p.last_nvec = (int)((p.row_bytes - (int64_t)(p.nchunks - 1) * kRwChunk) >> 4);
  // visiting stride: about half the row (the first two chunks are the sample), coprime to nchunks
  p.stride = p.nchunks / 2 > 1 ? p.nchunks / 2 : 1;
  auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
  while (gcd(p.stride, p.nchunks) != 1) ++p.stride;
  p.dense_noise = sp.noise.dense && (reinterpret_cast<uintptr_t>(sp.noise.dense) & 15) == 0 && (sp.noise.stride & 3) == 0;
  p.debug = (debug_stages() >> 4) & 7;
  int rc;
  if ((rc = ensure_smem((const void*)sample_rows_stream_kernel, kRwSmemBytes, "sample")) != TLX_OK) return rc;
  const int64_t cap = 2ll * sms;
  const int64_t grid = sp.rows < cap ? sp.rows : cap;
#ifdef TLX_TIMELINE
  p.sp.timeline = (long long*)sp.counters;   // timeline builds: the caller's workspace receives the stamps
#endif
  sample_rows_stream_kernel<<<(unsigned)grid, kRwThreads, kRwSmemBytes, st>>>(p);
  TLX_CHECK_LAUNCH("sample (rows)");
  return TLX_OK;
}

static int launch_stream_path(cudaStream_t st, const SampleParams& sp, void* workspace) {
  const StreamLayout l = stream_layout(sp.rows, sp.vocab);
  const int stages = debug_stages() & 15;
  unsigned char* ws = (unsigned char*)workspace;
  const int sms = device_sm_count();
  StreamParams p{};
  p.sp = sp;
  p.P = l.P; p.part_chunks = l.part_chunks; p.nchunks = l.nchunks; p.nfin = l.nfin; p.row_bytes = sp.vocab * 2;
  // the noise tensor can be streamed next to the logits if its rows start on 16-byte boundaries
  const int dense = sp.noise.dense && (reinterpret_cast<uintptr_t>(sp.noise.dense) & 15) == 0 && (sp.noise.stride & 3) == 0;
  // Wide rows' arg-max over their kept elements: with such a noise tensor the stream kernel does it (final
  // items, one record each; at most 128 per row); otherwise the finish kernel makes a final pass with the
  // CTAs that three per SM leave beside one per row.
  const int64_t fin_items = (sp.vocab + kStFinalElems - 1) / kStFinalElems;
  const bool final_in_stream = dense && fin_items <= 128 && fin_items <= l.nfin && !getenv("TLX_FINAL_IN_FINISH");
  p.fin_items = final_in_stream ? (int)fin_items : 0;
  p.fin_ctas = final_in_stream ? 0 : (3 * sms - (int)sp.rows < sms ? sms : 3 * sms - (int)sp.rows);
  p.error_flag = (int*)ws;
  p.item_counter = (int*)ws + 1;
  p.row_signals = (int*)ws + 2;
  p.desc = (StreamDesc*)(ws + l.off_desc);
  p.counts = (int*)(ws + l.off_counts);
  p.wlump = (double*)(ws + l.off_lump);
  p.wbest = (unsigned long long*)(ws + l.off_wbest);
  p.wflag = (int*)(ws + l.off_flag);
  p.rowdone = (int*)(ws + l.off_rowdone);
  p.wstate = (WideState*)(ws + l.off_state);
  p.records = (FinRecord*)(ws + l.off_records);
  p.whist = (uint32_t*)(ws + l.off_hist);
  p.cands = (uint32_t*)(ws + l.off_cands);
  p.debug = (debug_stages() >> 4) & 31;
  const int64_t items = sp.rows * (int64_t)l.P;
  const size_t st_smem = kStFixedSmem + (size_t)sp.rows * 6;   // descriptor word and order entry per row
  const size_t fin_smem = kStFinishFixedSmem + (size_t)sp.rows * sizeof(int);
  int rc;
  if ((rc = ensure_smem((const void*)sample_stream_kernel, st_smem, "sample")) != TLX_OK) return rc;
  if ((rc = ensure_smem((const void*)sample_finish_kernel, fin_smem, "sample")) != TLX_OK) return rc;
  // An SM changes its split between L1 and shared memory only while idle: the three kernels ask for the same
  // split, so that each one's CTAs can move in beside those of the one before.
  {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !done[dev]) {
      cudaFuncSetAttribute((const void*)sample_prologue_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      cudaFuncSetAttribute((const void*)sample_stream_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      cudaFuncSetAttribute((const void*)sample_finish_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      done[dev] = true;
    }
  }
#ifdef TLX_TIMELINE
  long long* tl = (long long*)(ws + l.off_timeline);
  p.sp.timeline = tl;
#define TLX_TIMELINE_KERNEL(k) p.sp.timeline = tl + (size_t)(k) * 8192 * 16
#else
#define TLX_TIMELINE_KERNEL(k) do {} while (0)
#endif
  sample_prologue_kernel<<<(unsigned)sp.rows, kStProThreads, 0, st>>>(p);
  TLX_CHECK_LAUNCH("sample (prologue)");
  if (stages < 2) return TLX_OK;
  const int64_t sgrid = items < 4ll * sms ? items : 4ll * sms;
  TLX_TIMELINE_KERNEL(1);
  if ((rc = launch_dependent(sample_stream_kernel, (unsigned)sgrid, kStThreads, st_smem, st, "sample (stream)", p)) != TLX_OK) return rc;
  if (stages < 3) return TLX_OK;
  TLX_TIMELINE_KERNEL(2);
  return launch_dependent(sample_finish_kernel, (unsigned)(p.fin_ctas + sp.rows), kStThreads, fin_smem, st,
                          "sample (finish)", p, dense);
}

}  // namespace tlx

using namespace tlx;

extern "C" {

size_t tlx_sample_workspace_bytes(int64_t rows, int64_t vocab) {
  if (rows <= 0 || vocab <= 0) return 0;
  const SliceLayout l = slice_layout(vocab, 4);  // the widest supported element
  const size_t sliced = counters_bytes(rows) + (size_t)rows * l.S * kRecordBytes;
  const size_t streamed = stream_layout(rows, vocab).bytes;
  return sliced > streamed ? sliced : streamed;
}

// Key and row offset of a call: host values or device operands (see NoiseSrc).
struct CallOperands {
  uint32_t key0 = 0, key1 = 0;
  int64_t dim0_offset = 0;
  const uint32_t* key_dev = nullptr;
  const int32_t* dim0_offset_dev = nullptr;
};

static int sample_impl(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab, int64_t row_stride,
                       const int32_t* top_k, const float* top_p, const float* temperature, const float* noise,
                       int64_t noise_stride, const CallOperands& op, int32_t* out_tokens, int32_t* out_status,
                       void* workspace, size_t workspace_bytes) {
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t key0 = op.key0, key1 = op.key1;
  const int64_t dim0_offset = op.dim0_offset;
  TLX_CHECK_ARG(rows >= 0 && vocab >= 1, "sample: bad extent");
  TLX_CHECK_ARG(vocab < (1ll << 31) && rows < (1ll << 31), "sample: extent too large");
  TLX_CHECK_ARG(row_stride >= vocab, "sample: row stride smaller than the row");
  if (dtype != TLX_F32 && dtype != TLX_BF16)
    return set_error(TLX_ERR_UNSUPPORTED, "sample: logits dtype %d not supported (f32, bf16)", dtype);
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(logits && top_k && top_p && temperature && out_tokens, "sample: null pointer");
  TLX_CHECK_ARG(!noise || noise_stride >= vocab, "sample: noise stride smaller than the row");
  const int es = dtype_bytes(dtype);
  const SliceLayout l = slice_layout(vocab, es);
  if (l.S > kMaxSlices)
    return set_error(TLX_ERR_UNSUPPORTED, "sample: vocabulary of %lld needs %d slices per row, at most %d supported",
                     (long long)vocab, l.S, kMaxSlices);
  TLX_CHECK_ARG(rows * (int64_t)l.S < (1ll << 30), "sample: too many work items");
  const size_t need = counters_bytes(rows) + (size_t)rows * l.S * kRecordBytes;
  if (!workspace || workspace_bytes < need)
    return set_error(TLX_ERR_WORKSPACE, "sample: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  TLX_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "sample: workspace must be 16-byte aligned");

  SampleParams p{};
  p.logits = logits; p.rows = rows; p.vocab = vocab; p.row_stride = row_stride;
  p.top_k = top_k; p.top_p = top_p; p.temperature = temperature;
  p.noise.dense = noise; p.noise.stride = noise_stride; p.noise.k0 = key0; p.noise.k1 = key1; p.noise.vocab = vocab;
  p.noise.key_dev = op.key_dev; p.noise.row_offset_dev = op.dim0_offset_dev;
  p.dim0_offset = dim0_offset; p.out_tokens = out_tokens; p.out_status = out_status;
  p.S = l.S; p.chunk_elems = l.chunk_elems; p.nchunks = l.nchunks;
  p.div_magic = ((1ull << 40) + (unsigned long long)l.S - 1) / (unsigned long long)l.S;
  // bulk copies need 16-byte aligned row starts and a row length that is a multiple of 16 bytes
  p.use_tma = ((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && ((row_stride * es) & 15) == 0 && ((vocab * es) & 15) == 0) ? 1 : 0;
  p.counters = (int32_t*)workspace;
  p.rowstate = reinterpret_cast<RowState*>((unsigned char*)workspace + 256);
  p.records = (unsigned char*)workspace + counters_bytes(rows);

  if (stream_path_serves(dtype, rows, vocab, row_stride, logits)) {
    // the rows are split over the CTAs; the row-per-CTA kernel is kept for comparison (diagnostic switch
    // TLX_SAMPLE_PATH=rows): it is faster on batches without wide rows and much slower with them
    const char* force = getenv("TLX_SAMPLE_PATH");
    const bool by_rows = force && force[0] == 'r';
    if (by_rows) return launch_rows_path(st, p);
    if (workspace_bytes >= stream_layout(rows, vocab).bytes) return launch_stream_path(st, p, workspace);
  }

  const int64_t items = rows * l.S;
  const int64_t slots = 2ll * device_sm_count();
  const int64_t wide_vecs_per_cta = ((vocab >> 3) + kWideCluster - 1) / kWideCluster;
  const bool resident_wide = 2 * rows >= slots && dtype == TLX_BF16 && p.use_tma && wide_vecs_per_cta * 16 <= kWidePartBytes;
  if (!resident_wide) {   // the flags in the workspace are only used by the slices kernel and its merges
    cudaError_t e = cudaMemsetAsync(workspace, 0, 256, st);
    if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "sample: cudaMemsetAsync: %s", cudaGetErrorString(e));
  }
  int rc;
  if (2 * rows >= slots) {
    // at least half a row per CTA slot: one CTA per row; only the rows whose top-k is disabled or
    // large are cut into slices first (their histograms need every SM), by the slices kernel
    const unsigned grid = (unsigned)(rows < slots ? rows : slots);
    if (resident_wide) {
      // rows without top-k: one cluster per row, the row resident in the cluster's shared memory
      if ((rc = ensure_smem((const void*)sample_wide_rows_kernel, kWideSmem, "sample")) != TLX_OK) return rc;
      if ((rc = ensure_smem((const void*)sample_rows_kernel<TLX_BF16>, kRowsSmem, "sample")) != TLX_OK) return rc;
      int64_t clusters = slots / kWideCluster;
      clusters = clusters < 1 ? 1 : (clusters > rows ? rows : clusters);
      // The two kernels work on disjoint rows: the cluster kernel goes to a side stream forked
      // from the caller's stream and joined back to it, so that they share the GPU.
      // (Only after tlx_init(device, TLX_INIT_SIDE_STREAM); otherwise both run on the caller's stream.)
      SideStream* side = side_stream();
      cudaStream_t wst = st;
      if (side && cudaEventRecord(side->fork, st) == cudaSuccess &&
          cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
        wst = side->stream;
      sample_wide_rows_kernel<<<(unsigned)(clusters * kWideCluster), kThreads, kWideSmem, wst>>>(p);
      const cudaError_t wide_err = cudaGetLastError();
      // whatever happens below, the caller's stream is joined to the side stream before this call returns
      bool joined = wst == st;
      if (!joined && cudaEventRecord(side->join, wst) == cudaSuccess) {
        if (wide_err == cudaSuccess) {
          p.wide_elsewhere = 1;
          sample_rows_kernel<TLX_BF16><<<grid, kRowsKThreads, kRowsSmem, st>>>(p);
        }
        joined = cudaStreamWaitEvent(st, side->join, 0) == cudaSuccess;
      } else if (joined && wide_err == cudaSuccess) {
        p.wide_elsewhere = 1;
        sample_rows_kernel<TLX_BF16><<<grid, kRowsKThreads, kRowsSmem, st>>>(p);
      }
      if (!joined) {
        // the events failed: wait for the side stream on the host, so that nothing of this call outlives it
        cudaStreamSynchronize(side->stream);
        cudaGetLastError();
        return set_error(TLX_ERR_CUDA, "sample: could not join the side stream");
      }
      if (wide_err != cudaSuccess)
        return set_error(TLX_ERR_CUDA, "sample (wide rows): launch failed: %s", cudaGetErrorString(wide_err));
    } else if (dtype == TLX_BF16) {
      p.only_general = 1;
      p.have_records = 1;
      const unsigned sgrid = (unsigned)(items < slots ? items : slots);
      if ((rc = ensure_smem((const void*)sample_slices_kernel<TLX_BF16>, kSlicesSmem, "sample")) != TLX_OK) return rc;
      if ((rc = ensure_smem((const void*)sample_rows_kernel<TLX_BF16>, kRowsSmem, "sample")) != TLX_OK) return rc;
      sample_slices_kernel<TLX_BF16><<<sgrid, kThreads, kSlicesSmem, st>>>(p);
      TLX_CHECK_LAUNCH("sample (slices)");
      sample_rows_kernel<TLX_BF16><<<grid, kRowsKThreads, kRowsSmem, st>>>(p);
      TLX_CHECK_LAUNCH("sample (rows)");
      p.final_pass = 1;   // rows without top-k: Gumbel arg-max over the kept elements, slice by slice
      sample_slices_kernel<TLX_BF16><<<sgrid, kThreads, kSlicesSmem, st>>>(p);
    } else {
      if ((rc = ensure_smem((const void*)sample_rows_kernel<TLX_F32>, kRowsSmem, "sample")) != TLX_OK) return rc;
      sample_rows_kernel<TLX_F32><<<grid, kRowsKThreads, kRowsSmem, st>>>(p);
    }
    TLX_CHECK_LAUNCH("sample (rows)");
    return TLX_OK;
  }
  // small batches: cut the rows into slices so that every SM streams, then merge per row
  const unsigned grid = (unsigned)(items < slots ? items : slots);
  if (dtype == TLX_BF16) {
    if ((rc = ensure_smem((const void*)sample_slices_kernel<TLX_BF16>, kSlicesSmem, "sample")) != TLX_OK) return rc;
    if ((rc = ensure_smem((const void*)sample_merge_kernel<TLX_BF16>, kMergeSmem, "sample")) != TLX_OK) return rc;
    sample_slices_kernel<TLX_BF16><<<grid, kThreads, kSlicesSmem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (slices)");
    sample_merge_kernel<TLX_BF16><<<(unsigned)rows, kRowThreads, kMergeSmem, st>>>(p);
  } else {
    if ((rc = ensure_smem((const void*)sample_slices_kernel<TLX_F32>, kSlicesSmem, "sample")) != TLX_OK) return rc;
    if ((rc = ensure_smem((const void*)sample_merge_kernel<TLX_F32>, kMergeSmem, "sample")) != TLX_OK) return rc;
    sample_slices_kernel<TLX_F32><<<grid, kThreads, kSlicesSmem, st>>>(p);
    TLX_CHECK_LAUNCH("sample (slices)");
    sample_merge_kernel<TLX_F32><<<(unsigned)rows, kRowThreads, kMergeSmem, st>>>(p);
  }
  TLX_CHECK_LAUNCH("sample");
  return TLX_OK;
}

int tlx_debug_check_status(int32_t* out4) {
#ifdef TLX_CHECKED
  int32_t w[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpyFromSymbol(w, g_tlx_check_word, sizeof(w)) != cudaSuccess)
    return set_error(TLX_ERR_CUDA, "debug_check_status: could not read the check word");
  const int32_t zero[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_tlx_check_word, zero, sizeof(zero));
  if (out4) for (int i = 0; i < 4; ++i) out4[i] = w[i];
  return w[0] ? 1 : 0;
#else
  if (out4) for (int i = 0; i < 4; ++i) out4[i] = 0;
  return set_error(TLX_ERR_UNSUPPORTED, "debug_check_status: not a checked build (python -m tallax_b200.build --checked)");
#endif
}

int tlx_init(int device, unsigned flags) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    return set_error(TLX_ERR_INVALID, "init: no CUDA device %d", device);
  int prev = 0;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return set_error(TLX_ERR_CUDA, "init: cudaSetDevice(%d) failed", device);
  device_sm_count();
  int rc = TLX_OK;
  if (flags & TLX_INIT_SIDE_STREAM) {
    if (side_stream(true)) g_side_stream_enabled.store(1);
    else rc = set_error(TLX_ERR_CUDA, "init: could not create the side stream");
  }
  cudaSetDevice(prev);
  return rc;
}

int tlx_sample(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab, int64_t row_stride,
               const int32_t* top_k, const float* top_p, const float* temperature, const float* noise,
               int64_t noise_stride, uint32_t key0, uint32_t key1, int64_t dim0_offset, int32_t* out_tokens,
               int32_t* out_status, void* workspace, size_t workspace_bytes) {
  CallOperands op;
  op.key0 = key0; op.key1 = key1; op.dim0_offset = dim0_offset;
  return sample_impl(stream, logits, dtype, rows, vocab, row_stride, top_k, top_p, temperature, noise, noise_stride, op,
                     out_tokens, out_status, workspace, workspace_bytes);
}

int tlx_sample_dev(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab, int64_t row_stride,
                   const int32_t* top_k, const float* top_p, const float* temperature, const float* noise,
                   int64_t noise_stride, const uint32_t* key_dev, const int32_t* dim0_offset_dev, int32_t* out_tokens,
                   int32_t* out_status, void* workspace, size_t workspace_bytes) {
  if (!noise && !key_dev) return set_error(TLX_ERR_INVALID, "sample: neither noise nor a key given");
  CallOperands op;
  op.key_dev = key_dev; op.dim0_offset_dev = dim0_offset_dev;
  return sample_impl(stream, logits, dtype, rows, vocab, row_stride, top_k, top_p, temperature, noise, noise_stride, op,
                     out_tokens, out_status, workspace, workspace_bytes);
}

static int top_p_and_sample_impl(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx, int64_t rows,
                                 int k, const float* top_p, const float* temperature, const float* noise,
                                 int64_t noise_stride, const CallOperands& op, int64_t vocab_size, double replace_val,
                                 int32_t* out_tokens) {
  const uint32_t key0 = op.key0, key1 = op.key1;
  const int64_t dim0_offset = op.dim0_offset;
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 0 && k >= 1, "top_p_and_sample: bad extent");
  if (k > 1024) return set_error(TLX_ERR_UNSUPPORTED, "top_p_and_sample: k=%d exceeds 1024", k);
  TLX_CHECK_ARG(vocab_size >= 1, "top_p_and_sample: vocab_size must be positive");
  if (rows == 0) return TLX_OK;
  TLX_CHECK_ARG(topk_logits && topk_idx && top_p && temperature && out_tokens, "top_p_and_sample: null pointer");
  NoiseSrc ns{noise, noise_stride, key0, key1, vocab_size, op.key_dev, op.dim0_offset_dev};
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

int tlx_top_p_and_sample(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx, int64_t rows,
                         int k, const float* top_p, const float* temperature, const float* noise,
                         int64_t noise_stride, uint32_t key0, uint32_t key1, int64_t vocab_size, double replace_val,
                         int64_t dim0_offset, int32_t* out_tokens) {
  CallOperands op;
  op.key0 = key0; op.key1 = key1; op.dim0_offset = dim0_offset;
  return top_p_and_sample_impl(stream, topk_logits, dtype, topk_idx, rows, k, top_p, temperature, noise, noise_stride, op,
                               vocab_size, replace_val, out_tokens);
}

int tlx_top_p_and_sample_dev(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx, int64_t rows,
                             int k, const float* top_p, const float* temperature, const float* noise,
                             int64_t noise_stride, const uint32_t* key_dev, int64_t vocab_size, double replace_val,
                             const int32_t* dim0_offset_dev, int32_t* out_tokens) {
  if (!noise && !key_dev) return set_error(TLX_ERR_INVALID, "top_p_and_sample: neither noise nor a key given");
  CallOperands op;
  op.key_dev = key_dev; op.dim0_offset_dev = dim0_offset_dev;
  return top_p_and_sample_impl(stream, topk_logits, dtype, topk_idx, rows, k, top_p, temperature, noise, noise_stride, op,
                               vocab_size, replace_val, out_tokens);
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

static int gumbel_argmax_impl(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1, int64_t rows,
                              int64_t cols, uint32_t key0, uint32_t key1, const uint32_t* key_dev, int64_t dim1_size,
                              int axis, int32_t* out_pos) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(axis == 0 || axis == 1, "gumbel_argmax: axis must be 0 or 1, got %d", axis);
  TLX_CHECK_ARG(rows > 0 && cols > 0 && dim1_size > 0, "gumbel_argmax: bad extent");
  TLX_CHECK_ARG(logits && idx0 && idx1 && out_pos, "gumbel_argmax: null pointer");
  const int64_t lines = axis == 1 ? rows : cols;
  gumbel_argmax_kernel<<<(unsigned)lines, 256, 0, st>>>(logits, idx0, idx1, rows, cols, key0, key1, key_dev, dim1_size,
                                                       axis, out_pos);
  TLX_CHECK_LAUNCH("gumbel_argmax");
  return TLX_OK;
}

int tlx_gumbel_argmax(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1, int64_t rows,
                      int64_t cols, uint32_t key0, uint32_t key1, int64_t dim1_size, int axis, int32_t* out_pos) {
  return gumbel_argmax_impl(stream, logits, idx0, idx1, rows, cols, key0, key1, nullptr, dim1_size, axis, out_pos);
}

int tlx_gumbel_argmax_dev(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1, int64_t rows,
                          int64_t cols, const uint32_t* key_dev, int64_t dim1_size, int axis, int32_t* out_pos) {
  if (!key_dev) return set_error(TLX_ERR_INVALID, "gumbel_argmax: null key");
  return gumbel_argmax_impl(stream, logits, idx0, idx1, rows, cols, 0u, 0u, key_dev, dim1_size, axis, out_pos);
}

static int launch_merge(cudaStream_t st, const MergeParams& p, int64_t rows) {
  int P = 2;
  while (P < p.n_cand) P <<= 1;
  const size_t smem = kSharedHeader + (size_t)P * 8 + (size_t)p.n_cand * 12;   // candidates, merged order, list
  int rc;
  if ((rc = ensure_smem((const void*)merge_and_sample_kernel, smem, "merge_and_sample")) != TLX_OK) return rc;
  // one thread per two (padded) candidates: the sort's stages pair them up, the tail takes two items per thread
  int threads = P / 2;
  threads = threads < 64 ? 64 : (threads > kMergeThreads ? kMergeThreads : threads);
  // many rows of few candidates: CTAs of 128 threads, eight per SM, so that a thousand rows are one wave
  if (rows >= 256 && P <= 1024 && threads > 128) threads = 128;
  if (p.xbuf) {
    // exchange mode: the rows' arrival counts order this kernel after the candidate kernels, so it may be
    // scheduled while this rank's candidate kernel still runs (its CTAs have all started by then) and has
    // its launch latency behind it when the first rows arrive
    return launch_dependent(merge_and_sample_kernel, (unsigned)rows, (unsigned)threads, smem, st, "merge_and_sample", p);
  }
  merge_and_sample_kernel<<<(unsigned)rows, threads, smem, st>>>(p);
  TLX_CHECK_LAUNCH("merge_and_sample");
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
  MergeParams p{};
  p.cand_vals = cand_vals; p.cand_idx = cand_idx; p.cand_noise = cand_noise; p.n_cand = n_cand;
  p.k_per_block = k_per_block; p.block_stride = block_stride; p.row_stride = row_stride; p.top_k = top_k;
  p.top_p = top_p; p.temperature = temperature; p.out = out_tokens;
  return launch_merge(st, p, rows);
}

int tlx_exchange_merge_and_sample(void* stream, void* exchange, int64_t rows, int k_cand, int world,
                                  const int32_t* top_k, const float* top_p, const float* temperature,
                                  int32_t* out_tokens, int32_t* out_status) {
  cudaStream_t st = (cudaStream_t)stream;
  TLX_CHECK_ARG(rows >= 1 && k_cand >= 1 && world >= 1 && world <= kExchangeMaxWorld, "exchange_merge_and_sample: bad extent");
  if ((int64_t)world * k_cand > kMergeMaxCand)
    return set_error(TLX_ERR_UNSUPPORTED, "exchange_merge_and_sample: %lld candidates exceed %d",
                     (long long)world * k_cand, kMergeMaxCand);
  TLX_CHECK_ARG(exchange && top_k && top_p && temperature && out_tokens, "exchange_merge_and_sample: null pointer");
  const ExchangeLayout l = exchange_layout(rows, k_cand, world);
  MergeParams p{};
  p.n_cand = world * k_cand; p.k_per_block = k_cand; p.block_stride = (int64_t)l.block_elems; p.row_stride = k_cand;
  p.top_k = top_k; p.top_p = top_p; p.temperature = temperature; p.out = out_tokens;
  p.xbuf = (unsigned char*)exchange; p.world = world; p.rows = rows; p.status = out_status;
  for (int q = 0; q < 2; ++q) { p.off_flags[q] = l.off_flags[q]; p.off_cand[q] = l.off_cand[q]; }
  return launch_merge(st, p, rows);
}

}  // extern "C"
