// Streaming form of the fused sampler for bf16 logits whose rows start on 16-byte boundaries.
// Included by sampler.cu (it uses that file's parameter block, PTX wrappers and row tails).
//
// A row is cut into at most 16 PARTS of a few 12 KB chunks; a work item is one (row, part).  Three
// kernels, chained by programmatic dependent launches (each starts while its predecessor drains and
// waits for the predecessor's results where it first needs them):
//
//   prologue  one CTA per row.  Reads the row's parameters and a 4096-element sample of the row
//             (16 segments spread over it) and leaves a descriptor: the row's class and
//               normal (1 <= top_k <= 1024, or greedy): the 16-bit key threshold that, with four
//                   standard deviations of margin, keeps at least top_k elements of the row;
//               wide   (top-k disabled, top_p < 1): the top of the histogram window, 512 keys (four
//                   binades) above the sample's maximum;
//               other  (anything else): answered by the whole-row routines in the finish kernel.
//   stream    persistent CTAs, 4 per SM; every CTA starts on the item of its own index and claims
//             further ones from a counter, one item ahead of need.  Wide rows' items come first (they
//             take longest).  Chunks arrive through a three-slot ring of bulk copies (cp.async.bulk +
//             mbarrier) that runs ahead across item boundaries.  Normal items: one packed compare per
//             16-byte vector, the warp notes the vectors that hold something, looks at them densely
//             (one element per lane) and appends (bits, position) to its own segment of the item's
//             candidate list in the workspace.  Wide items: histogram of the 16-bit keys inside the
//             window and sum of exp(x - window top) of everything below it, both added to the row's
//             totals in the workspace; the CTA that delivers a wide row's last part takes the row's
//             maximum, softmax denominator and top-p threshold key from the totals.
//   finish    two kinds of CTA in one grid.  The first ones stream the wide rows again, one CTA per
//             (row, range of 8 KB chunks), logits (from L2) and the chunk's noise side by side:
//             screened Gumbel score of every kept element; each range leaves its best element as a
//             record, and the CTA that delivers a row's last record decides the row on the
//             f64-evaluated term among the records within the screening slack of the best one.  The
//             other CTAs, one per row, finish the normal rows from their candidate lists (they were all
//             taken with the same threshold, so "at least top_k of them" proves that they hold the
//             top-k set): top-k boundary, softmax mass and top-p threshold from one histogram over the
//             candidates' keys, Gumbel arg-max over the kept ones.  A row whose threshold was too high,
//             whose lists overflowed or whose window did not settle it takes the exact whole-row
//             routines right there.
#pragma once

namespace tlx {

constexpr int kStThreads = 256;
constexpr int kStWarps = kStThreads / 32;
constexpr int kStChunk = 12288;                      // bytes per bulk copy and ring slot
constexpr int kStChunkElems = kStChunk / 2;          // bf16
constexpr int kStChunkVecs = kStChunk / 16;
constexpr int kStSlots = 3;
constexpr int kStVecPerThread = kStChunkVecs / kStThreads;    // 3
constexpr int kStMaxParts = 16;                      // parts per row
constexpr int kStMaxPartChunks = 10;                 // 61440 elements: a position inside a part fits 16 bits
constexpr int kStWarpCap = 128;                      // candidates one warp may publish per item
constexpr int kStSpec = 32;                          // entries of a segment the finish kernel fetches before it knows the count
constexpr int kStMaxK = 1024;                        // largest top_k served by the candidate lists
constexpr int kStWinExtra = 512;                     // window top = sample maximum + this many keys
constexpr int kStWin = kWin + kStWinExtra;           // bins per wide row in the workspace
constexpr int kStMaxRows = 8192;                     // per row 6 bytes of shared memory in the stream kernel
constexpr int kStSampleVecs = 4;                     // 16-byte vectors per prologue thread
constexpr int kStProThreads = 128;
constexpr int kStSample = kStProThreads * kStSampleVecs * 8;   // 4096 elements
constexpr int kStMinVocab = 16384;
constexpr int kFinChunk = 8192;                      // final pass: bytes of logits per slot ...
constexpr int kFinChunkElems = kFinChunk / 2;
constexpr int kFinNoiseChunk = kFinChunkElems * 4;   // ... and of f32 noise
// final items of the stream kernel: the logits and the noise of kStFinalElems elements of a wide row, in
// chunks that fill a slot of the ring (2 + 4 bytes per element)
constexpr int kStFinalChunkElems = kStChunk / 6;
constexpr int kStFinalChunks = 4;
constexpr int kStFinalElems = kStFinalChunks * kStFinalChunkElems;
constexpr int kFinSlots = 2;
constexpr int kFinVecPerThread = kFinChunk / 16 / kStThreads;   // 2
static_assert(kStMaxPartChunks * kStChunkElems <= 65536, "candidate positions are 16 bits");
static_assert(kStChunkVecs % kStThreads == 0 && kFinChunk / 16 % kStThreads == 0, "whole vectors per thread");
static_assert(kStMaxParts * kStWarps * (kStSpec / 16) <= kStThreads, "one round of speculative fetches per thread");

enum StClass : int { kStNormal = 0, kStWide = 1, kStOther = 2 };

struct __align__(16) StreamDesc {
  int cls;
  int K;        // effective top-k (1 for greedy rows)
  int key16;    // normal: candidate threshold; wide: top of the histogram window
  float xref;   // wide: value of the window top, the reference of the below-window sums
};

struct __align__(16) WideState {
  int result;                // kWideNotReady until the row's threshold is settled; then -1 (the window did not
                             // settle it) or (key of the greatest element - threshold key) << 16 | threshold key:
                             // an element is kept if its value is not below the value of the threshold key
  uint32_t best_key;         // best screened score of a kept element of the row known so far (ordered key):
                             // seeded with the score of the row's greatest element when the threshold is
                             // published (one 8-byte store with `result`), raised by the final items
  int parts_done;            // stream kernel: parts of the row whose totals are in
  int done;                  // final items (stream kernel) or ranges (finish kernel) that have delivered their record
};
static_assert(sizeof(WideState) == 16, "WideState layout");
constexpr int kWideNotReady = (int)0x80000000;
__device__ __forceinline__ int wide_result(int kmax16, int vstar16) {
  return vstar16 < 0 ? -1 : ((kmax16 - vstar16) << 16) | vstar16;
}
__device__ __forceinline__ int wide_vstar16(int result) { return result < 0 ? -1 : (result & 0xFFFF); }
__device__ __forceinline__ int wide_kmax16(int result) { return (result & 0xFFFF) + (result >> 16); }

struct __align__(16) FinRecord {   // best element of one range of chunks of a wide row
  float a;          // its screened score
  float u;          // its noise
  int tok;          // its token, 0x7FFFFFFF if the range has no kept element
  uint32_t bits;    // its bf16 bits | 0x10000 if other elements of the range come within the slack
};

struct StreamParams {
  SampleParams sp;
  int P;                 // parts per row
  int part_chunks;       // chunks per part (the row's last part may have fewer)
  int nchunks;           // stream chunks per row (the last one may be short)
  int nfin;              // final-pass chunks per row
  int fin_ctas;          // finish kernel: CTAs of the final pass (the first ones of the grid)
  int64_t row_bytes;
  StreamDesc* desc;      // [rows]
  int* counts;           // [rows * P * 8] candidates published per item and warp (may exceed kStWarpCap: overflow)
  uint32_t* cands;       // [rows * P * 8 * kStWarpCap] bf16 bits << 16 | position inside the part
  uint32_t* whist;       // [rows * kStWin] wide rows: window histogram, bin = window top - key16
  double* wlump;         // [rows * P] wide rows: sum of exp(x - xref) below the window
  unsigned long long* wbest;   // [rows] wide rows: (window top - key of the greatest element) << 32 | its token
  int* wflag;            // [rows] wide rows: an element lay above the window
  WideState* wstate;     // [rows]
  FinRecord* records;    // [rows * nfin]
  int fin_items;             // final items per wide row (kStFinalElems elements each); 0: the finish
                             // kernel makes the final pass over the wide rows
  int* rowdone;              // per row: parts of a normal row whose candidate lists are complete
  int* row_signals;          // 1 once the stream kernel has decided to count them (it does when the batch has
                             // wide rows, whose final items keep it busy long after the normal rows are done)
  int* item_counter;     // [1] next unclaimed item - gridDim.x (cleared by the prologue)
  int* error_flag;       // [1] a bounded wait of the stream kernel gave up (cleared by the prologue)
  int debug;             // diagnostic switches, 0 in normal use
};

// ---- bf16 bit helpers -------------------------------------------------------------------------
// Order-preserving 16-bit key of a bf16 bit pattern: -0 folded onto +0, every NaN the greatest key
// (the upper half of f32_key of the widened value).
__device__ __forceinline__ uint32_t bf16_key16(uint32_t b) {
  uint32_t k = (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
  k = (b & 0x7FFFu) > 0x7F80u ? 0xFFFFu : k;
  return b == 0x8000u ? 0x8000u : k;
}
__device__ __forceinline__ uint32_t key16_bf16_bits(uint32_t k) { return (k & 0x8000u) ? (k & 0x7FFFu) : (~k & 0xFFFFu); }
__device__ __forceinline__ __nv_bfloat162 bf162_splat_bits(uint32_t b16) { return bf162_bits(b16 | (b16 << 16)); }
// mbarrier wait that lets the hardware suspend the thread for up to about a microsecond per attempt
// instead of spinning on the issue slots; bounded like mbar_wait.
__device__ __forceinline__ bool mbar_wait_suspended(unsigned long long* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// Adds to a counter in global memory with release semantics at GPU scope: every write that this thread has
// made or has observed through a CTA barrier is visible to a thread that then reads the new count.  One
// instruction; the thread does not wait for the writes itself (a fence followed by a relaxed add would).
__device__ __forceinline__ void red_release_add(int* ptr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }

// Scratch of wide_threshold_core (up to 16 warps).
struct __align__(16) WideScratch {
  double dsum[16];
  double dlump[16];
  int first[16];
  int vstar;
  int kmax16;   // out: key of the greatest element
  int pad[2];
};

// Small per-CTA scratch shared by the kernels' block-wide steps.
struct __align__(16) StControl {
  unsigned long long mbar[4];
  int fifo[8];            // stream: items in the order the producer took them (row << 8 | part), -1 = no more
  int cnt;
  int flag;
  int vstar;
  uint32_t best_key;      // final pass: the CTA's best screened score so far, as an ordered key
  int pending[8];         // stream: rows of the normal items finished but not yet counted in rowdone (thread 0)
  int fin_result;         // final item: the row's WideState::result
  float fin_T;            // ... and temperature
  double dsum[kStWarps];
  double dlump[kStWarps];
  uint32_t wkey[kStWarps];
  int wtok[kStWarps];
  float fbest[kStWarps];
  int ibest[kStWarps];
  WideScratch wide;
};

constexpr size_t kStRingBytes = (size_t)kStSlots * kStChunk;
constexpr size_t kStAreaBytes = (size_t)kStWin * 4;          // a wide row's window
constexpr size_t kStListBytes = (size_t)kStWarps * (32 * kStVecPerThread) * 2;
constexpr size_t kStFixedSmem = kStRingBytes + kStAreaBytes + kStListBytes + sizeof(StControl);   // + 6 bytes per row

// Top-p threshold key of a wide row from its window histogram `hist` (kStWin bins in shared memory, bin i
// = key (window top - i)) and the sum of exp(x - value of the window top) below the window, of which every
// thread passes a share.  Returns -1 if the window does not settle it (bad_thread set by some thread: an
// element above the window or a NaN; a maximum too far below the window top; a threshold below the
// window).  All NT threads call; thread t owns the bins [t * kStWin / NT, (t + 1) * kStWin / NT).
template <int NT>
__device__ __forceinline__ int wide_threshold_core(int wtop, float pp, const uint32_t* hist, double lump_thread,
                                                       int bad_thread, WideScratch& ws) {
  constexpr int kPer = kStWin / NT;   // ascending i = descending key
  constexpr int kNW = NT / 32;
  static_assert(kStWin % NT == 0 && kNW <= 16, "window bins per thread");
  const int lane = lane_id(), warp = warp_id();
  const int i0 = threadIdx.x * kPer;
  int first = kStWin;   // lowest occupied bin among this thread's own
#pragma unroll 1
  for (int j = kPer - 1; j >= 0; --j)
    if (hist[i0 + j]) first = i0 + j;
  first = __reduce_min_sync(0xFFFFFFFFu, first);
  if (lane == 0) ws.first[warp] = first;
  const int bad = __syncthreads_or(bad_thread);
  int shift = ws.first[0];
#pragma unroll
  for (int w = 1; w < kNW; ++w) shift = min(shift, ws.first[w]);
  if (bad || shift > kStWinExtra) return -1;
  const int kmax16 = wtop - shift;
  const float xmax = key16_value(kmax16);
  double lm = 0.0;
#pragma unroll 1
  for (int j = 0; j < kPer; ++j) {
    const int i = i0 + j;
    const uint32_t c = hist[i];
    if (c && i >= shift && wtop - i >= 0) lm += (double)c * (double)expf(key16_value(wtop - i) - xmax);
  }
  double im = lm, il = lump_thread;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double nm = shfl_up_f64(im, o);
    if (lane >= o) im += nm;
    il += shfl_xor_f64(il, o);
  }
  if (lane == 31) { ws.dsum[warp] = im; ws.dlump[warp] = il; }
  if (threadIdx.x == 0) { ws.vstar = -1; ws.kmax16 = kmax16; }
  __syncthreads();
  double total = 0.0, below = 0.0;
  for (int w = 0; w < kNW; ++w) {
    if (w < warp) im += ws.dsum[w];
    total += ws.dsum[w];
    below += ws.dlump[w];
  }
  if (below > 0.0) total += below * exp((double)key16_value(wtop) - (double)xmax);
  const double target = (double)pp * total;
  const double em = im - lm;
  if (em < target && im >= target) {
    double run = em;
#pragma unroll 1
    for (int j = 0; j < kPer; ++j) {
      const int i = i0 + j;
      const uint32_t c = hist[i];
      if (c && i >= shift && wtop - i >= 0) {
        run += (double)c * (double)expf(key16_value(wtop - i) - xmax);
        if (run >= target) { ws.vstar = wtop - i; break; }
      }
    }
  }
  __syncthreads();
  return ws.vstar;
}

// The same for a row of the split-row path, whose sums below the window sit in the workspace, one per part.
static __device__ __forceinline__ int st_wide_threshold(const StreamParams& p, int row, int wtop, float pp,
                                                        const uint32_t* hist, WideScratch& ws) {
  double lump = 0.0;
  int bad = __ldcg(p.wflag + row) != 0;
  if ((int)threadIdx.x < p.P) {
    lump = __ldcg(p.wlump + (size_t)row * p.P + threadIdx.x);
    if (!(lump >= 0.0)) { bad = 1; lump = 0.0; }   // a NaN below the window
  }
  return wide_threshold_core<kStThreads>(wtop, pp, hist, lump, bad, ws);
}

// A row's class as far as its parameters decide it (the prologue may still turn a row into kStOther on
// what it finds in the row's sample).  K_out: the effective top-k.
__device__ __forceinline__ int st_param_class(int top_k, float pp, float T_, int64_t V, int& K_out) {
  int K = top_k;
  if (K <= 0 || (int64_t)K >= V) K = (int)V;
  if (T_ < kSamplingEps) K = 1;   // greedy: the top candidate
  K_out = K;
  if (K <= kStMaxK) {
    // rank in the sample that leaves, with four standard deviations of margin, at least K elements of the
    // row at or above the sample's element of that rank: too many candidates -> whole-row routines
    const float mu = (float)K * (float)kStSample / (float)V;
    const int r = (int)(mu + 4.0f * sqrtf(mu) + 2.999f);
    return (float)r * (float)V / (float)kStSample > 0.8f * (float)kMergeCap ? kStOther : kStNormal;
  }
  return ((int64_t)K >= V && pp < 1.0f) ? kStWide : kStOther;
}

// ---- prologue ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kStProThreads) sample_prologue_kernel(StreamParams p) {
  __shared__ int red[2][kStProThreads / 32];
  const int row = blockIdx.x;
  const int lane = lane_id(), warp = warp_id();
  const int64_t V = p.sp.vocab;
  const __nv_bfloat16* rowp = reinterpret_cast<const __nv_bfloat16*>(p.sp.logits) + (int64_t)row * p.sp.row_stride;
  TLX_STAMP(p.sp, 0);
  // the stream kernel may start now: it requests its first copies and then waits for this kernel's end
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the sample: 16 segments of 32 vectors, evenly spread over the row's full vectors
  const uint4* vp = reinterpret_cast<const uint4*>(rowp);
  const int64_t nv = V >> 3;
  uint4 sv[kStSampleVecs];
#pragma unroll
  for (int j = 0; j < kStSampleVecs; ++j) {
    const int g = j * (kStProThreads / 32) + warp;
    const int64_t start = ((int64_t)g * (nv - 32)) / (kStSampleVecs * (kStProThreads / 32) - 1);
    sv[j] = __ldg(vp + start + lane);
  }
  const float T_ = p.sp.temperature[row];
  const float pp = p.sp.top_p[row];
  int K;
  int cls = st_param_class(p.sp.top_k[row], pp, T_, V, K);

  __nv_bfloat162 h[kStSampleVecs * 4];
#pragma unroll
  for (int j = 0; j < kStSampleVecs; ++j) {
    h[4 * j + 0] = bf162_bits(sv[j].x); h[4 * j + 1] = bf162_bits(sv[j].y);
    h[4 * j + 2] = bf162_bits(sv[j].z); h[4 * j + 3] = bf162_bits(sv[j].w);
  }
  int key16 = 0;
  float xref = 0.f;
  if (cls == kStNormal) {
    // rank in the sample that leaves, with four standard deviations of margin, at least K elements
    // of the row at or above the sample's element of that rank
    const float mu = (float)K * (float)kStSample / (float)V;
    int r = (int)(mu + 4.0f * sqrtf(mu) + 2.999f);
    r = r > kStSample ? kStSample : r;
    // largest key t (not a NaN key) with #(sample >= t) >= r: sixteen halvings, counted with packed compares
    int lo = 0, hi = 0xFF81;
    for (int round = 0; round < 16 && hi - lo > 1; ++round) {
      const int mid = (lo + hi) >> 1;
      const __nv_bfloat162 t2 = bf162_splat_bits(key16_bf16_bits((uint32_t)mid));
      __nv_bfloat162 acc4[4] = {bf162_bits(0u), bf162_bits(0u), bf162_bits(0u), bf162_bits(0u)};
#pragma unroll
      for (int i = 0; i < kStSampleVecs * 4; ++i) acc4[i & 3] = __hadd2(acc4[i & 3], __hgeu2(h[i], t2));
      const __nv_bfloat162 acc = __hadd2(__hadd2(acc4[0], acc4[1]), __hadd2(acc4[2], acc4[3]));
      int c = (int)(__low2float(acc) + __high2float(acc) + 0.5f);
      c = __reduce_add_sync(0xFFFFFFFFu, c);
      if (lane == 0) red[round & 1][warp] = c;
      __syncthreads();
      int total = 0;
#pragma unroll
      for (int w = 0; w < kStProThreads / 32; ++w) total += red[round & 1][w];
      if (total >= r) lo = mid; else hi = mid;
    }
    key16 = lo;
  } else if (cls == kStWide) {
    __nv_bfloat162 m = h[0];
#pragma unroll
    for (int i = 1; i < kStSampleVecs * 4; ++i) m = __hmax2_nan(m, h[i]);
    const uint32_t mb = *reinterpret_cast<uint32_t*>(&m);
    const uint32_t k0 = bf16_key16(mb & 0xFFFFu), k1 = bf16_key16(mb >> 16);
    int km = (int)(k0 > k1 ? k0 : k1);
    km = __reduce_max_sync(0xFFFFFFFFu, km);
    if (lane == 0) red[0][warp] = km;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kStProThreads / 32; ++w) km = max(km, red[0][w]);
    if (km > 0xFF80) {
      cls = kStOther;   // a NaN in the sample: the whole-row routines know what to do
      if (threadIdx.x == 0) {   // the stream kernel lists the row by its parameters: its final items see "unsettled"
        WideState ws{};
        ws.result = -1;
        p.wstate[row] = ws;
      }
    } else {
      key16 = min(km + kStWinExtra, 0xFF80);
      xref = key16_value(key16);
      uint4* wh = reinterpret_cast<uint4*>(p.whist + (size_t)row * kStWin);
      for (int i = threadIdx.x; i < kStWin / 4; i += kStProThreads) wh[i] = make_uint4(0, 0, 0, 0);
      if (threadIdx.x == 0) {
        p.wflag[row] = 0;
        p.wbest[row] = ~0ull;
        WideState ws{};
        ws.result = kWideNotReady;
        ws.best_key = f32_key(-INFINITY);
        p.wstate[row] = ws;
      }
    }
  }
  if (threadIdx.x == 0) {
    StreamDesc d;
    d.cls = cls; d.K = K; d.key16 = key16; d.xref = xref;
    p.desc[row] = d;
    p.rowdone[row] = 0;
    if (p.sp.out_status) p.sp.out_status[row] = 0;
    if (row == 0) { *p.error_flag = 0; *p.item_counter = 0; *p.row_signals = 0; }
  }
  TLX_STAMP(p.sp, 1);
}

// ---- stream: per-chunk workers -------------------------------------------------------------------
// Normal rows.  wl: this warp's list of the chunk's vectors that may hold a candidate.  A candidate is
// an element that is not below the threshold value (a NaN is one); it is stored as its bf16 bits and
// its position inside the part, in the warp's own segment of the item's list in the workspace (dst,
// wc entries so far).  kFull: the chunk has all of its vectors.
template <bool kFull>
__device__ __forceinline__ void st_filter_chunk(const unsigned char* buf, int nvec, int pos0, float tvf,
                                                __nv_bfloat162 tv2, uint32_t* dst, int& wc, unsigned short* wl) {
  const int lane = lane_id();
  const uint32_t lt = (1u << lane) - 1u;
  int wn = 0;
#pragma unroll
  for (int j = 0; j < kStVecPerThread; ++j) {
    const int v = (int)threadIdx.x + j * kStThreads;
    bool hit = false;
    if (kFull || v < nvec) {
      const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
      const __nv_bfloat162 m =
          __hmax2_nan(__hmax2_nan(bf162_bits(x.x), bf162_bits(x.y)), __hmax2_nan(bf162_bits(x.z), bf162_bits(x.w)));
      hit = !__hblt2(m, tv2);   // some element is not below the threshold value
    }
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, hit);
    if (mask) {
      if (hit && TLX_IN_BOUNDS(wn + __popc(mask & lt), 32 * kStVecPerThread, 1)) wl[wn + __popc(mask & lt)] = (unsigned short)v;
      wn += __popc(mask);
    }
  }
  if (wn == 0) return;
  __syncwarp();
  for (int base = 0; base < wn; base += 4) {
    const int e = base + (lane >> 3);
    bool pass = false;
    uint32_t entry = 0;
    if (e < wn) {
      const int q = wl[e] * 8 + (lane & 7);
      const uint32_t bits = TLX_IN_BOUNDS(q, kStChunkElems, 2) ? reinterpret_cast<const unsigned short*>(buf)[q] : 0u;
      pass = !(__uint_as_float(bits << 16) < tvf) && TLX_IN_BOUNDS(pos0 + q, 65536, 3);   // positions are 16 bits
      entry = (bits << 16) | (uint32_t)(pos0 + q);
    }
    const uint32_t pm = __ballot_sync(0xFFFFFFFFu, pass);
    const int pos = wc + __popc(pm & lt);
    if (pass && pos < kStWarpCap) dst[pos] = entry;
    wc += __popc(pm);
  }
  __syncwarp();
}

// Wide rows: window histogram (bin = window top - key; -0 keeps its own key, one below +0's, which the
// tail treats as the same value) and the sum below the window.  `above` collects the sign of
// (window top - key): negative once an element lies above the window (a positive NaN does).
// No branches: every element computes its bin and its exp; predicates pick what is used.
template <bool kFull, int NT = kStThreads, int VPT = kStVecPerThread>
__device__ __forceinline__ void st_hist_chunk(const unsigned char* buf, int nvec, int wtop, float nxl, uint32_t* win,
                                              float& lump, int& above, int pos0, uint32_t& dmin) {
#pragma unroll 1
  for (int j = 0; j < VPT; ++j) {
    const int v = (int)threadIdx.x + j * NT;
    if (kFull || v < nvec) {
      const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      int d[8];
      float val[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t hi = (e & 1) ? (w[e >> 1] & 0xFFFF0000u) : (w[e >> 1] << 16);   // the element as f32 bits
        const uint32_t sgn = (uint32_t)((int32_t)hi >> 31);
        const uint32_t k16 = (hi >> 16) ^ ((sgn & 0x7FFFu) | 0x8000u);
        d[e] = wtop - (int)k16;
        val[e] = ex2_approx(fmaf(__uint_as_float(hi), 1.44269504f, nxl));
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        above |= d[e];
        dmin = min(dmin, ((uint32_t)d[e] << 16) | (uint32_t)(pos0 + v * 8 + e));   // greatest key, with its position
        if ((unsigned)d[e] < (unsigned)kStWin) atomicAdd(&win[d[e]], 1u);
        lump += d[e] >= kStWin ? val[e] : 0.f;
      }
    }
  }
}

// The producer's state (thread 0): the item whose chunks are being requested, and the one claimed for
// afterwards (its value is first used an item later, so the counter's round trip stays off the path).
// The list of items is built from the rows' parameters (no need to wait for the prologue kernel): a CTA's
// first item is the one of its own index, so its copies are requested before anything about the rows'
// contents is known; further items are claimed from a counter.  Rows of class "other" are not streamed.
constexpr int kStClaimLate = -2;   // StProducer::next: no item claimed ahead, claim when one is needed
struct StProducer {
  int item;    // >= 0: there is an item (its code); -1: no more
  int row, part, chunk, nchunks;
  int next;    // claimed index (0, 1, ... among the claimed items)
  int pushed;
};

// Item codes: row << 8 | part for the logits of a part of a row; row << 8 | 0x80 | sub for a final item
// (logits and noise of the elements [sub * kStFinalElems, (sub + 1) * kStFinalElems) of a wide row).
struct StOrder {
  const unsigned short* rows;   // the wide rows, then the normal rows (each in row order)
  int nwide;
  int nwide_items, nnormal_items, nfinal_items;
  // item index -> code, or -1 past the end.  Order: the wide rows' histogram items (every CTA's first item
  // is taken by its index, so these start at once, at most one per CTA while there are CTAs enough: the rows'
  // thresholds are what the final items wait for), the normal rows' items, the final items.
  __device__ __forceinline__ int item(int j, int P, int fin_items) const {
    if (j < nwide_items) {
      const int r = j / P;
      return ((int)rows[r] << 8) | (j - r * P);
    }
    j -= nwide_items;
    if (j < nnormal_items) {
      const int r = j / P;
      return ((int)rows[nwide + r] << 8) | (j - r * P);
    }
    j -= nnormal_items;
    if (j >= nfinal_items) return -1;
    const int w = j / fin_items;
    return ((int)rows[w] << 8) | 0x80 | (j - w * fin_items);
  }
};

__device__ __forceinline__ int st_part_chunks(const StreamParams& p, int part) {
  const int rest = p.nchunks - part * p.part_chunks;
  return rest < p.part_chunks ? rest : p.part_chunks;
}
__device__ __forceinline__ int st_final_item_chunks(const StreamParams& p, int sub) {
  const int64_t rest = p.sp.vocab - (int64_t)sub * kStFinalElems;
  return rest >= kStFinalElems ? kStFinalChunks : (int)((rest + kStFinalChunkElems - 1) / kStFinalChunkElems);
}
__device__ __forceinline__ int st_code_chunks(const StreamParams& p, int code) {
  return (code & 0x80) ? st_final_item_chunks(p, code & 0x7F) : st_part_chunks(p, code & 0x7F);
}

__device__ __forceinline__ void st_issue_chunk(const StreamParams& p, StProducer& ps, unsigned char* ring, StControl& ctl,
                                               int slot) {
  const unsigned char* src;
  uint32_t bytes;
  if (ps.part & 0x80) {
    // logits to the front of the slot, noise behind them
    const int64_t e0 = (int64_t)(ps.part & 0x7F) * kStFinalElems + (int64_t)ps.chunk * kStFinalChunkElems;
    const int64_t rest = p.sp.vocab - e0;
    const uint32_t elems = (uint32_t)(rest < kStFinalChunkElems ? rest : kStFinalChunkElems);
    unsigned char* dst = ring + (size_t)slot * kStChunk;
    mbar_expect_tx(&ctl.mbar[slot], elems * 6);
    bulk_load(dst, reinterpret_cast<const __nv_bfloat16*>(p.sp.logits) + (int64_t)ps.row * p.sp.row_stride + e0, elems * 2,
              &ctl.mbar[slot]);
    bulk_load(dst + kStFinalChunkElems * 2, p.sp.noise.dense_row(ps.row + p.sp.dim0_offset) + e0,
              elems * 4, &ctl.mbar[slot]);
    ps.chunk++;
    return;
  } else {
    const int c = ps.part * p.part_chunks + ps.chunk;
    const int64_t off = (int64_t)c * kStChunk;
    const int64_t rest = p.row_bytes - off;
    bytes = (uint32_t)(rest < kStChunk ? rest : kStChunk);
    src = reinterpret_cast<const unsigned char*>(p.sp.logits) + (int64_t)ps.row * p.sp.row_stride * 2 + off;
  }
  mbar_expect_tx(&ctl.mbar[slot], bytes);
  bulk_load(ring + (size_t)slot * kStChunk, src, bytes, &ctl.mbar[slot]);
  ps.chunk++;
}

// Requests the next chunk into `slot` (thread 0 only).
__device__ __forceinline__ void st_issue(const StreamParams& p, StProducer& ps, const StOrder& order, unsigned char* ring,
                                         StControl& ctl, int slot) {
  for (;;) {
    if (ps.item < 0) return;
    if (ps.chunk < ps.nchunks) break;
    if (ps.next == kStClaimLate) ps.next = (int)gridDim.x + atomicAdd(p.item_counter, 1);
    const int code = order.item(ps.next, p.P, p.fin_items);
    ps.item = code;
    if (code >= 0) {
      ps.row = code >> 8;
      ps.part = code & 0xFF;
      ps.chunk = 0;
      ps.nchunks = st_code_chunks(p, code);
      // The next item is claimed now, an item ahead, so that the counter's round trip stays off the path --
      // except behind a final item when there are fewer final items than CTAs: those are the last items of
      // the list and long ones, and a CTA that holds one must not sit on a second one while other CTAs run
      // out of work.  (With many final items per CTA claiming late would leave the ring dry at every item.)
      ps.next = ((code & 0x80) && order.nfinal_items <= (int)gridDim.x) ? kStClaimLate
                                                                        : (int)gridDim.x + atomicAdd(p.item_counter, 1);
    }
    ctl.fifo[ps.pushed & 7] = code;
    ps.pushed++;
  }
  st_issue_chunk(p, ps, ring, ctl, slot);
}

// A chunk of a final item: logits (front of the slot) and noise (behind them) of the elements [elem0,
// elem0 + 8 ngroups) of a wide row; a thread takes one group of eight.  Kept elements (value not below
// tvf) whose noise passes the test below are scored.
// The test: with cbm = (a score that some kept element of the row reaches) - margin, an element of value x
// and noise u can come within the screening slack of the row's best score only if x / T + g(u) >= cbm,
// g = -log(-log u); since -log u >= 1 - u that needs 1 - u <= exp(-(cbm - x / T)).  It is made once per
// group with the group's greatest value, which only loosens it.
// Per thread: the best two screened scores of the item so far (a1 >= a2), with the best one's noise, bf16
// bits and token.
__device__ __forceinline__ void st_final_chunk(const unsigned char* buf, int ngroups, int elem0, __nv_bfloat162 tv2,
                                               float tvf, float inv_T, float cbm, float& a1, float& a2, float& u1,
                                               uint32_t& b1, int& t1) {
  const int v = (int)threadIdx.x;
  if (v >= ngroups) return;
  const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
  const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(x.x), bf162_bits(x.y)), __hmax2_nan(bf162_bits(x.z), bf162_bits(x.w)));
  if (__hblt2(m, tv2)) return;   // all eight below the threshold
  const float xg = fmaxf(__low2float(m), __high2float(m));   // NaN-propagating max: a NaN keeps the test open
  const float eps = xg == xg ? __expf(-(cbm - xg * inv_T)) * 1.00001f : INFINITY;
  const float* nbuf = reinterpret_cast<const float*>(buf + kStFinalChunkElems * 2) + v * 8;
  const float4 n0 = *reinterpret_cast<const float4*>(nbuf);
  const float4 n1 = *reinterpret_cast<const float4*>(nbuf + 4);
  const float umax = fmaxf(fmaxf(fmaxf(n0.x, n0.y), fmaxf(n0.z, n0.w)), fmaxf(fmaxf(n1.x, n1.y), fmaxf(n1.z, n1.w)));
  if (1.0f - umax > eps) return;   // none of the eight can matter
  const unsigned short* xb = reinterpret_cast<const unsigned short*>(buf) + v * 8;
#pragma unroll 1
  for (int e = 0; e < 8; ++e) {
    const float u = nbuf[e];
    const uint32_t bits = xb[e];
    const float xf = __uint_as_float(bits << 16);
    if (!(xf < tvf) && 1.0f - u <= eps) {
      const float a = fmaf(xf, inv_T, gumbel_screen(u));
      const int tok = elem0 + v * 8 + e;
      if (a > a1 || (a == a1 && tok < t1)) { a2 = a1; a1 = a; u1 = u; b1 = bits; t1 = tok; }
      else if (a > a2) a2 = a;
    }
  }
}

// Counts the noted items in their rows' rowdone (thread 0): one fence for all of them, then plain adds.
__device__ __forceinline__ int st_publish_rows(const StreamParams& p, StControl& ctl, int n) {
  if (n > 0) {
    __threadfence();
    for (int i = 0; i < n; ++i) atomicAdd(&p.rowdone[ctl.pending[i]], 1);
  }
  return 0;
}

// Shared memory beyond the fixed part: per row 4 bytes of descriptor (class << 16 | key) and 2 bytes of order.
// The grid is a multiple of P (whole rows in the first wave) and at most rows * P.
__global__ void __launch_bounds__(kStThreads, 4) sample_stream_kernel(StreamParams p) {
  extern __shared__ __align__(128) unsigned char st_smem[];
  unsigned char* ring = st_smem;
  uint32_t* area = reinterpret_cast<uint32_t*>(st_smem + kStRingBytes);
  unsigned short* wl =
      reinterpret_cast<unsigned short*>(st_smem + kStRingBytes + kStAreaBytes) + warp_id() * (32 * kStVecPerThread);
  StControl& ctl = *reinterpret_cast<StControl*>(st_smem + kStRingBytes + kStAreaBytes + kStListBytes);
  uint32_t* dtab = reinterpret_cast<uint32_t*>(st_smem + kStFixedSmem);
  unsigned short* order_rows = reinterpret_cast<unsigned short*>(dtab + p.sp.rows);
  const int rows = (int)p.sp.rows;
  const int lane = lane_id(), warp = warp_id();
  TLX_STAMP(p.sp, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStSlots; ++s) mbar_init(&ctl.mbar[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The list of rows needs the rows' classes only as far as the parameters decide them (a row that the
  // prologue downgrades is dropped when its items come up): it is built while the prologue kernel still runs.
  uint32_t* pcls = dtab;   // parameter classes, replaced by the descriptors below
  for (int r = threadIdx.x; r < rows; r += kStThreads) {
    int K;
    pcls[r] = (uint32_t)st_param_class(p.sp.top_k[r], p.sp.top_p[r], p.sp.temperature[r], p.sp.vocab, K);
  }
  __syncthreads();
  int nlisted = 0, nwide = 0;
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const uint32_t want = pass == 0 ? (uint32_t)kStWide : (uint32_t)kStNormal;
#pragma unroll 1
    for (int base = 0; base < rows; base += kStThreads) {
      const int r = base + (int)threadIdx.x;
      const bool take = r < rows && pcls[r] == want;
      const uint32_t mask = __ballot_sync(0xFFFFFFFFu, take);
      if (lane == 0) ctl.ibest[warp] = __popc(mask);
      __syncthreads();
      int off = nlisted, total = 0;
#pragma unroll 1
      for (int w = 0; w < kStWarps; ++w) {
        if (w < warp) off += ctl.ibest[w];
        total += ctl.ibest[w];
      }
      if (take && TLX_IN_BOUNDS(off + __popc(mask & ((1u << lane) - 1u)), rows, 10))
        order_rows[off + __popc(mask & ((1u << lane) - 1u))] = (unsigned short)r;
      nlisted += total;
      __syncthreads();
    }
    if (pass == 0) nwide = nlisted;
  }
  StOrder order;
  order.rows = order_rows;
  order.nwide = nwide;
  order.nwide_items = nwide * p.P;
  order.nnormal_items = (nlisted - nwide) * p.P;
  order.nfinal_items = nwide * p.fin_items;
  // the CTA's first item, and its first copies
  StProducer ps;
  ps.item = order.item((int)blockIdx.x, p.P, p.fin_items);
  ps.row = ps.item >> 8;
  ps.part = ps.item & 0xFF;
  ps.chunk = 0;
  ps.nchunks = ps.item >= 0 ? st_code_chunks(p, ps.item) : 0;
  ps.next = 0;
  ps.pushed = 1;
  if (threadIdx.x == 0) {
    ctl.fifo[0] = ps.item;
    for (int s = 0; s < kStSlots && s < ps.nchunks; ++s) st_issue_chunk(p, ps, ring, ctl, s);
  }
  // everything below reads what the prologue kernel wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The finish kernel's CTAs move in as these leave.  Released only here, after the wait: a finish CTA then
  // starts after the prologue kernel has completed, and may read the rows' descriptors and completion
  // counters without waiting for this whole kernel.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  TLX_STAMP(p.sp, 6);
  if (threadIdx.x == 0) ps.next = (int)gridDim.x + atomicAdd(p.item_counter, 1);
  for (int r = threadIdx.x; r < rows; r += kStThreads) {
    const StreamDesc d = p.desc[r];
    dtab[r] = ((uint32_t)d.cls << 16) | (uint32_t)d.key16;
  }
  __syncthreads();
  TLX_STAMP(p.sp, 7);
  // Counting the rows' finished parts costs the producer thread a fence per item: worth it only when final
  // items will keep this kernel busy after the normal rows are complete.
  const bool signal_rows = order.nfinal_items > 0;
  if (signal_rows && blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<volatile int*>(p.row_signals) = 1;
  if (threadIdx.x == 0) {
    // a first item shorter than the ring: go on into the claimed items
    for (int s = ps.chunk; s < kStSlots; ++s) st_issue(p, ps, order, ring, ctl, s);
  }
  __syncthreads();

  const int last_nvec = (int)((p.row_bytes - (int64_t)(p.nchunks - 1) * kStChunk) >> 4);
  int slot = 0;
  uint32_t phase = 0;
  int taken = 0;   // items this CTA has started
  int npending = 0;   // thread 0: entries of ctl.pending
  TLX_STAMP(p.sp, 1);
  for (int code = ctl.fifo[0]; code >= 0; code = ctl.fifo[taken & 7]) {
    ++taken;
    const int row = code >> 8, part = code & 0x7F;
    if (code & 0x80) {
      // ---- a final item: the Gumbel arg-max over the kept elements of a range of a wide row
      if (threadIdx.x == 0) {
        npending = st_publish_rows(p, ctl, npending);
        // the row's threshold: settled by whoever brought the last part of its histogram.  Those items were
        // all claimed before this one, by CTAs that wait for nothing but their copies, so the wait is
        // short; it is bounded all the same.
#ifdef TLX_TIMELINE
        const long long tl_f0 = global_timer_ns();
        if (p.sp.timeline && p.sp.timeline[(size_t)blockIdx.x * 16 + 13] == 0) p.sp.timeline[(size_t)blockIdx.x * 16 + 13] = tl_f0;
#endif
        volatile unsigned long long* rp = reinterpret_cast<volatile unsigned long long*>(&p.wstate[row]);
        const float T_ = p.sp.temperature[row];   // one round trip for both loads
        unsigned long long w = *rp;               // result and best score, published as one word
        for (int spin = 0; (int)(uint32_t)w == kWideNotReady && spin < (1 << 16); ++spin) {
          __nanosleep(64);
          w = *rp;
        }
        int res = (int)(uint32_t)w;
        if (res == kWideNotReady) { *p.error_flag = 1; res = -1; }
        ctl.fin_result = res;
        ctl.best_key = (uint32_t)(w >> 32);
        ctl.fin_T = T_;
#ifdef TLX_TIMELINE
        if (p.sp.timeline) { p.sp.timeline[(size_t)blockIdx.x * 16 + 12] += 1; p.sp.timeline[(size_t)blockIdx.x * 16 + 14] += global_timer_ns() - tl_f0; }
#endif
      }
      __syncthreads();
      const int res = ctl.fin_result;
      const float inv_T = 1.0f / ctl.fin_T;
      const uint32_t tbits = key16_bf16_bits((uint32_t)wide_vstar16(res));
      const __nv_bfloat162 tv2 = bf162_splat_bits(tbits);
      const float tvf = __uint_as_float(tbits << 16);
      const int nc = st_final_item_chunks(p, part);
      const int64_t last_elems = p.sp.vocab - ((int64_t)part * kStFinalElems + (int64_t)(nc - 1) * kStFinalChunkElems);
      float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f, published = -INFINITY;
      uint32_t b1 = 0;
      int t1 = 0x7FFFFFFF;
      for (int ci = 0; ci < nc; ++ci) {
        // the best score known so far, less twice the screening slack (see st_final_chunk)
        const float cb = key_f32(ctl.best_key);
        const float cbm = cb - 2.0f * (kGumbelSlack + 1e-5f * fabsf(cb));
        const bool arrived = mbar_wait_suspended(&ctl.mbar[slot], phase);
        const unsigned char* buf = ring + (size_t)slot * kStChunk;
        const int elem0 = part * kStFinalElems + ci * kStFinalChunkElems;
        if (res >= 0 && !(p.debug & 1)) {
          const int ngroups = ci != nc - 1 || last_elems >= kStFinalChunkElems ? kStFinalChunkElems / 8 : (int)(last_elems >> 3);
          st_final_chunk(buf, ngroups, elem0, tv2, tvf, inv_T, cbm, a1, a2, u1, b1, t1);
        }
        if (a1 > published) { atomicMax(&ctl.best_key, f32_key(a1)); published = a1; }
        if (__syncthreads_or(!arrived)) {
          if (threadIdx.x == 0) *p.error_flag = 1;
          return;
        }
        if (threadIdx.x == 0) st_issue(p, ps, order, ring, ctl, slot);
        if (++slot == kStSlots) { slot = 0; phase ^= 1u; }
      }
#ifdef TLX_TIMELINE
      if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 15] = global_timer_ns() - p.sp.timeline[(size_t)blockIdx.x * 16 + 13];
#endif
      if (res >= 0) {
        // the item's record: its best element, and whether anything else of it comes within the slack
        const uint32_t key = f32_key(a1);
        const uint32_t wkey = __reduce_max_sync(0xFFFFFFFFu, key);
        const int wtok = __reduce_min_sync(0xFFFFFFFFu, key == wkey ? t1 : 0x7FFFFFFF);
        if (lane == 0) { ctl.wkey[warp] = wkey; ctl.wtok[warp] = wtok; }
        __syncthreads();
        uint32_t bkey = ctl.wkey[0];
        int btok = ctl.wtok[0];
#pragma unroll 1
        for (int i = 1; i < kStWarps; ++i) {
          const uint32_t k = ctl.wkey[i];
          const int tk = ctl.wtok[i];
          if (k > bkey || (k == bkey && tk < btok)) { bkey = k; btok = tk; }
        }
        const bool any = btok != 0x7FFFFFFF;
        const bool mine = any ? (key == bkey && t1 == btok) : threadIdx.x == 0;
        const float amax = key_f32(bkey);
        const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
        const int multi = __syncthreads_or(any && ((!mine && a1 >= cut) || a2 >= cut));
        if (mine) {
          FinRecord r;
          r.a = a1; r.u = u1; r.tok = any ? t1 : 0x7FFFFFFF; r.bits = b1 | (multi ? 0x10000u : 0u);
          if (TLX_IN_BOUNDS(part, p.nfin, 8) && TLX_IN_BOUNDS(row, rows, 9)) p.records[(size_t)row * p.nfin + part] = r;
          if (any) atomicMax(&p.wstate[row].best_key, bkey);
        }
      }
      __syncthreads();   // the producer's fifo entries are visible; ctl is free again
      // the item's record (if any) is in: the row's finish CTA counts the items
      if (threadIdx.x == 0) red_release_add(&p.wstate[row].done, 1);
#ifdef TLX_TIMELINE
      if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 9] = global_timer_ns() - p.sp.timeline[(size_t)blockIdx.x * 16 + 13];
#endif
      if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 5] = taken * 16 + 3;
      continue;
    }
    const uint32_t dw = TLX_IN_BOUNDS(row, rows, 7) ? dtab[row] : ((uint32_t)kStOther << 16);
    const int cls = (int)(dw >> 16), key16 = (int)(dw & 0xFFFFu);
    const int c0 = part * p.part_chunks;
    const int nc = st_part_chunks(p, part);
    const uint32_t tbits = key16_bf16_bits((uint32_t)key16);
    const __nv_bfloat162 tv2 = bf162_splat_bits(tbits);
    const float tvf = __uint_as_float(tbits << 16);
    const float nxl = -tvf * 1.44269504f;   // wide rows: tvf is the value of the window top
    const size_t seg = ((size_t)row * p.P + part) * kStWarps + warp;   // this warp's segment of the item's list
    uint32_t* dst = p.cands + seg * kStWarpCap;
    int wc = 0;
    float lump = 0.f;
    int above = 0;
    uint32_t dmin = 0xFFFFFFFFu;   // wide rows: (window top - key) << 16 | position in the part, of the greatest element
    if (cls == kStWide) {
      for (int i = threadIdx.x; i < kStWin; i += kStThreads) area[i] = 0;
      __syncthreads();
    }
    for (int ci = 0; ci < nc; ++ci) {
      const bool arrived = mbar_wait_suspended(&ctl.mbar[slot], phase);
      if (taken == 1 && ci == 0) TLX_STAMP(p.sp, 2);
      const unsigned char* buf = ring + (size_t)slot * kStChunk;
      const bool full = c0 + ci != p.nchunks - 1;
      if (p.debug & 1) {
      } else if (cls == kStNormal) {
        if (full) st_filter_chunk<true>(buf, kStChunkVecs, ci * kStChunkElems, tvf, tv2, dst, wc, wl);
        else st_filter_chunk<false>(buf, last_nvec, ci * kStChunkElems, tvf, tv2, dst, wc, wl);
      } else if (cls == kStWide) {
        if (full) st_hist_chunk<true>(buf, kStChunkVecs, key16, nxl, area, lump, above, ci * kStChunkElems, dmin);
        else st_hist_chunk<false>(buf, last_nvec, key16, nxl, area, lump, above, ci * kStChunkElems, dmin);
      }
      if (__syncthreads_or(!arrived)) {   // a copy never arrived: give up, the finish kernel reports it
        if (threadIdx.x == 0) *p.error_flag = 1;
        return;
      }
      // the chunk is consumed, its slot is free
      if (threadIdx.x == 0) st_issue(p, ps, order, ring, ctl, slot);
      if (++slot == kStSlots) { slot = 0; phase ^= 1u; }
    }
#ifdef TLX_TIMELINE
    long long tl_t = global_timer_ns();
#endif
    if (cls == kStNormal) {
      if (lane == 0) p.counts[seg] = wc;
    } else if (cls == kStWide) {
      // this part's totals go to the row's; the CTA that brings the last part settles the row's threshold
      uint32_t* gh = p.whist + (size_t)row * kStWin;
      for (int i = threadIdx.x; i < kStWin; i += kStThreads) {
        const uint32_t c = area[i];
        if (c) atomicAdd(&gh[i], c);
      }
      double l = (double)lump;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += shfl_xor_f64(l, o);
      dmin = __reduce_min_sync(0xFFFFFFFFu, dmin);
      if (lane == 0) { ctl.dsum[warp] = l; ctl.wkey[warp] = dmin; }
      if (above < 0) p.wflag[row] = 1;
      __syncthreads();   // with thread 0's fence below: every thread's additions come before the count
      if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kStWarps; ++w) t += ctl.dsum[w];
        p.wlump[(size_t)row * p.P + part] = t;
        uint32_t dm = ctl.wkey[0];
        for (int w = 1; w < kStWarps; ++w) dm = min(dm, ctl.wkey[w]);
        atomicMin(&p.wbest[row], ((unsigned long long)(dm >> 16) << 32) |
                                     (unsigned long long)((uint32_t)part * (uint32_t)(p.part_chunks * kStChunkElems) + (dm & 0xFFFFu)));
        __threadfence();
        ctl.flag = atomicAdd(&p.wstate[row].parts_done, 1) == p.P - 1;
      }
      __syncthreads();
#ifdef TLX_TIMELINE
      if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 8] = global_timer_ns() - tl_t;
#endif
      if (ctl.flag) {
        __threadfence();
        for (int i = threadIdx.x; i < kStWin; i += kStThreads) area[i] = __ldcg(gh + i);
        __syncthreads();
#ifdef TLX_TIMELINE
        if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 10] = global_timer_ns() - tl_t;
#endif
        const int v = st_wide_threshold(p, row, key16, p.sp.top_p[row], area, ctl.wide);
        if (threadIdx.x == 0) {
          // The row's greatest element is always kept: its screened score (the very expression its final item
          // will evaluate) seeds the row's best score, so that the final items' test bites from their first
          // chunk on.  Threshold and seed become visible together (one 8-byte store).
          uint32_t seed = f32_key(-INFINITY);
          const unsigned long long wb = __ldcg(&p.wbest[row]);
          const int64_t pos = (int64_t)(uint32_t)wb;
          const float T_ = p.sp.temperature[row];
          if (v >= 0 && p.fin_items > 0 && pos < p.sp.vocab && (wb >> 32) < 65536ull) {
            const uint32_t bits = reinterpret_cast<const unsigned short*>(p.sp.logits)[(int64_t)row * p.sp.row_stride + pos];
            const float u = p.sp.noise.at(row + p.sp.dim0_offset, pos);
            seed = f32_key(fmaf(__uint_as_float(bits << 16), 1.0f / T_, gumbel_screen(u)));
          }
          const unsigned long long word = ((unsigned long long)seed << 32) | (unsigned long long)(uint32_t)wide_result(ctl.wide.kmax16, v);
          *reinterpret_cast<volatile unsigned long long*>(&p.wstate[row]) = word;
        }
#ifdef TLX_TIMELINE
        if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 11] = global_timer_ns() - tl_t;
#endif
      }
    }
    __syncthreads();   // the producer's fifo entries are visible; the shared window is free again
    if (signal_rows && cls == kStNormal && threadIdx.x == 0) {
      // This part's candidates and counts are written (all warps, before the barrier).  The row's finish CTA
      // waits for the count of finished parts; publishing it needs a release, which holds this thread (the
      // producer) up for a round trip, so finished items are noted and published together: when the list is
      // full, before a final item, at the end.  Finish CTAs find room only when CTAs of this kernel leave.
      ctl.pending[npending++] = row;
      if (npending == 8) npending = st_publish_rows(p, ctl, npending);
    }
    if (taken == 1) TLX_STAMP(p.sp, 3);
    if (threadIdx.x == 0 && p.sp.timeline) p.sp.timeline[(size_t)blockIdx.x * 16 + 5] = taken * 16 + cls;
  }
  if (threadIdx.x == 0) st_publish_rows(p, ctl, npending);
  TLX_STAMP(p.sp, 4);
}

// ---- finish: normal rows from their candidate lists -------------------------------------------------
constexpr int kTlBins = 4096;   // keys above the candidate threshold that the histogram tail can tell apart
constexpr int kTlSegs = kStMaxParts * kStWarps;   // (item, warp) segments of a row

// Shared memory of a finish CTA while it finishes a normal row on the short path.  It overlays the
// SelectShared + candidate area that the whole-row routines use when the short path does not apply,
// and the final pass's ring.
struct __align__(16) TailShared {
  uint32_t hist[kTlBins];          // candidates per key, bin = key16 - threshold key
  uint32_t tok[kMergeCap];         // the candidates' tokens ...
  unsigned short key[kMergeCap];   // ... and keys
  uint32_t raw[kTlSegs * kStSpec]; // the segments' first kStSpec entries as fetched (32 slots per segment)
  int segcnt[kTlSegs];
  int segoff[kTlSegs];             // exclusive offsets of the segments
  uint32_t scan_c[kStWarps];
  double scan_m[kStWarps];
  double Z;
  int m, bad, maxbin, overflow;
  int vk_idx, admitted, ties_total, vstar_idx;
  int nties, pad;
  uint32_t wkey[kStWarps];
  int wtok[kStWarps];
};

// Block-wide (max score, lowest token) over one candidate per thread; valid in every thread.
__device__ __forceinline__ void tl_block_top(float a, int tok, TailShared& t, uint32_t& bkey, int& btok) {
  const uint32_t key = f32_key(a);
  const uint32_t wkey = __reduce_max_sync(0xFFFFFFFFu, key);
  const int wtok = __reduce_min_sync(0xFFFFFFFFu, key == wkey ? tok : 0x7FFFFFFF);
  __syncthreads();
  if (lane_id() == 0) { t.wkey[warp_id()] = wkey; t.wtok[warp_id()] = wtok; }
  __syncthreads();
  bkey = t.wkey[0];
  btok = t.wtok[0];
#pragma unroll
  for (int i = 1; i < kStWarps; ++i) {
    const uint32_t k = t.wkey[i];
    const int tk = t.wtok[i];
    if (k > bkey || (k == bkey && tk < btok)) { bkey = k; btok = tk; }
  }
}

// One candidate of segment `sg` goes to position f of the shared arrays and into the histogram.
__device__ __forceinline__ void tl_place(TailShared& t, const StreamParams& p, const StreamDesc& d, const float* noise_row,
                                         uint32_t e, int sg, int f, int& mymax, int& over) {
  const uint32_t k16 = bf16_key16(e >> 16);
  const int bin = (int)k16 - d.key16;
  const uint32_t tok = (uint32_t)(sg / kStWarps) * (uint32_t)(p.part_chunks * kStChunkElems) + (e & 0xFFFFu);
  if (!TLX_IN_BOUNDS(f, kMergeCap, 4) || !TLX_IN_BOUNDS(tok, p.sp.vocab, 5)) return;
  t.tok[f] = tok;
  t.key[f] = (unsigned short)k16;
  if (noise_row) prefetch_l2(noise_row + tok);   // most candidates' noise is wanted a few microseconds from now
  if (bin >= 0 && bin < kTlBins) { atomicAdd(&t.hist[bin], 1u); mymax = max(mymax, bin); }
  else over = 1;
}

// Finishes a normal row from its candidate lists: top-k boundary, softmax mass over the top-k set,
// top-p threshold (all from one histogram over the candidates' keys: the mass of a value group is
// count * exp(value - max)), then the Gumbel arg-max over the kept candidates.  Returns the token, or
// -1 if the lists cannot be trusted to hold the row's top-K or the keys spread over more than kTlBins
// values (the caller then takes the whole-row routines).  All threads call; hist[] must be zero.
// What a thread of a row CTA fetches of the row's candidate lists in the first round trip: thread =
// (segment, half); the count of the segment and every second 16-byte vector of its first kStSpec entries.
struct TailFetch {
  uint4 e[4];
  int cnt;
};
__device__ __forceinline__ TailFetch tl_fetch(const StreamParams& p, int row) {
  constexpr int kSubs = kStSpec / 16;
  const int nseg = p.P * kStWarps;
  const int sg = (int)threadIdx.x / kSubs, sub = (int)threadIdx.x % kSubs;
  TailFetch r;
  r.cnt = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) r.e[q] = make_uint4(0, 0, 0, 0);
  if (sg < nseg) {
    r.cnt = __ldcg(p.counts + (size_t)row * nseg + sg);
    const uint4* src = reinterpret_cast<const uint4*>(p.cands + ((size_t)row * nseg + sg) * kStWarpCap) + sub;
#pragma unroll
    for (int q = 0; q < 4; ++q) r.e[q] = __ldcg(src + q * kSubs);
  }
  return r;
}

__device__ __forceinline__ int st_finish_normal(const StreamParams& p, int row, const StreamDesc& d, float pp, float T_,
                                                    const TailFetch& fetched, TailShared& t) {
  const SampleParams& sp = p.sp;
  const int K = d.K;
  const int nseg = p.P * kStWarps;
  const int lane = lane_id(), warp = warp_id();
  const int64_t nrow = row + sp.dim0_offset;
  const float* noise_row = sp.noise.dense ? sp.noise.dense_row(nrow) : nullptr;
  // ---- one round trip: every segment's count and its first kStSpec entries (thread = segment and half)
  constexpr int kSubs = kStSpec / 16;   // threads per segment
  const uint32_t* cbase = p.cands + (size_t)row * nseg * kStWarpCap;
  const int sg = (int)threadIdx.x / kSubs, sub = (int)threadIdx.x % kSubs;
  const int cnt = fetched.cnt;
  if (sg < nseg) {
    if (sub == 0) t.segcnt[sg] = cnt;
    uint4* rv = reinterpret_cast<uint4*>(t.raw) + sg * (kStSpec / 4) + sub;
#pragma unroll
    for (int q = 0; q < 4; ++q) rv[q * kSubs] = fetched.e[q];
  }
  if (threadIdx.x == 0) { t.maxbin = 0; t.overflow = 0; t.nties = 0; }
  __syncthreads();
  // ---- the segments' offsets (warp 0: four segments per lane)
  if (warp == 0) {
    int c[4], sum = 0, bad = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int sg = lane * 4 + q;
      c[q] = sg < nseg ? t.segcnt[sg] : 0;
      if (c[q] > kStWarpCap) bad = 1;
      sum += c[q];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += n;
    }
    int off = incl - sum;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int sg = lane * 4 + q;
      if (sg < nseg) t.segoff[sg] = off;
      off += c[q];
    }
    bad = __any_sync(0xFFFFFFFFu, bad);
    if (lane == 31) { t.m = incl; t.bad = bad; }
  }
  __syncthreads();
  const int m = t.m;
  if (t.bad || m > kMergeCap || m < K) return -1;
  TLX_STAMP(sp, 2);
  // ---- candidates: tokens and keys to shared memory, keys into the histogram
  {
    int mymax = 0, over = 0;
    // The fetched slots, dealt evenly to the threads (a slot is an entry if its index is below its segment's
    // count).  Rolled on purpose, as are the loops below: this code runs once per CTA, so the time goes into
    // fetching its instructions, not into executing them.
#pragma unroll 2
    for (int i = threadIdx.x; i < nseg * kStSpec; i += kStThreads) {
      const int s2 = i / kStSpec, idx = i % kStSpec;
      if (idx < t.segcnt[s2]) tl_place(t, p, d, noise_row, t.raw[i], s2, t.segoff[s2] + idx, mymax, over);
    }
    // what a segment holds beyond the entries fetched ahead: a warp per such segment
#pragma unroll 1
    for (int s2 = warp; s2 < nseg; s2 += kStWarps) {
      const int c = t.segcnt[s2];
      for (int idx = kStSpec + lane; idx < c; idx += 32)
        tl_place(t, p, d, noise_row, __ldcg(cbase + (size_t)s2 * kStWarpCap + idx), s2, t.segoff[s2] + idx, mymax, over);
    }
    mymax = __reduce_max_sync(0xFFFFFFFFu, mymax);
    if (lane == 0) atomicMax(&t.maxbin, mymax);
    if (over) t.overflow = 1;
  }
  __syncthreads();
  if (t.overflow) return -1;
  TLX_STAMP(sp, 3);
  if (T_ < kSamplingEps) {
    // greedy: the greatest key, lowest token
    uint32_t bk = 0;
    int bt = 0x7FFFFFFF;
    for (int f = threadIdx.x; f < m; f += kStThreads) {
      const uint32_t k = t.key[f];
      const int tk = (int)t.tok[f];
      if (k > bk || (k == bk && tk < bt)) { bk = k; bt = tk; }
    }
    const uint32_t wk = __reduce_max_sync(0xFFFFFFFFu, bk);
    const int wt = __reduce_min_sync(0xFFFFFFFFu, bk == wk ? bt : 0x7FFFFFFF);
    if (lane == 0) { t.wkey[warp] = wk; t.wtok[warp] = wt; }
    __syncthreads();
    uint32_t k0 = t.wkey[0];
    int t0 = t.wtok[0];
    for (int i = 1; i < kStWarps; ++i)
      if (t.wkey[i] > k0 || (t.wkey[i] == k0 && t.wtok[i] < t0)) { k0 = t.wkey[i]; t0 = t.wtok[i]; }
    return t0;
  }
  // ---- one scan over the bins in descending key order: counts and (unbounded) mass
  const int maxbin = t.maxbin;
  const int W = maxbin + 1;
  const int kmax16 = d.key16 + maxbin;
  const float xmax = key16_value(kmax16);
  const int per = (W + kStThreads - 1) / kStThreads;
  const int i0 = threadIdx.x * per;   // idx = maxbin - bin
  uint32_t lc = 0;
  double lm = 0.0;
#pragma unroll 1
  for (int j = 0; j < per; ++j) {
    const int idx = i0 + j;
    if (idx < W) {
      const uint32_t c = t.hist[maxbin - idx];
      if (c) { lc += c; lm += (double)c * (double)expf(key16_value(kmax16 - idx) - xmax); }
    }
  }
  uint32_t ic = lc;
  double im = lm;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nc = __shfl_up_sync(0xFFFFFFFFu, ic, o);
    const double nm = shfl_up_f64(im, o);
    if (lane >= o) { ic += nc; im += nm; }
  }
  if (lane == 31) { t.scan_c[warp] = ic; t.scan_m[warp] = im; }
  __syncthreads();
  for (int w = 0; w < warp; ++w) { ic += t.scan_c[w]; im += t.scan_m[w]; }
  const uint32_t ec = ic - lc;   // exclusive prefixes
  const double em = im - lm;
  if (ec < (uint32_t)K && ic >= (uint32_t)K) {
    // the top-k boundary lies in this thread's bins
    uint32_t run = ec;
    double mass = em;
#pragma unroll 1
    for (int j = 0; j < per; ++j) {
      const int idx = i0 + j;
      const uint32_t c = t.hist[maxbin - idx];
      const double ex = (double)expf(key16_value(kmax16 - idx) - xmax);
      if (run + c >= (uint32_t)K) {
        t.vk_idx = idx;
        t.admitted = (int)((uint32_t)K - run);
        t.ties_total = (int)c;
        t.Z = mass + (double)((uint32_t)K - run) * ex;
        t.vstar_idx = idx;   // default: the whole top-k set is kept
        break;
      }
      run += c;
      mass += (double)c * ex;
    }
  }
  __syncthreads();
  const int vk_idx = t.vk_idx, admitted = t.admitted, ties_total = t.ties_total;
  const double target = (double)pp * t.Z;
  if (em < target && i0 <= vk_idx) {
    // first value group at which the cumulative mass over the top-k set reaches top_p * Z
    double run = em;
#pragma unroll 1
    for (int j = 0; j < per; ++j) {
      const int idx = i0 + j;
      if (idx > vk_idx) break;
      const uint32_t c = idx == vk_idx ? (uint32_t)admitted : t.hist[maxbin - idx];
      if (c) {
        run += (double)c * (double)expf(key16_value(kmax16 - idx) - xmax);
        if (run >= target) { t.vstar_idx = idx; break; }
      }
    }
  }
  __syncthreads();
  const int vstar_idx = t.vstar_idx;
  const bool cut_ties = vstar_idx == vk_idx && admitted < ties_total;
  TLX_STAMP(sp, 5);
  // the lowest tokens of the boundary group are the admitted ones: list the group's tokens, then mark
  // (top bit of the token) the group's members beyond the admitted ones
  uint32_t* tie_tok = t.hist;   // the histogram is no longer needed
  if (cut_ties) {
    __syncthreads();
#pragma unroll 1
    for (int f = threadIdx.x; f < m; f += kStThreads)
      if (kmax16 - (int)t.key[f] == vk_idx) {
        const int slot = atomicAdd(&t.nties, 1);
        if (TLX_IN_BOUNDS(slot, kTlBins, 6)) tie_tok[slot] = t.tok[f];
      }
    __syncthreads();
    const int nties = t.nties;
#pragma unroll 1
    for (int f = threadIdx.x; f < m; f += kStThreads) {
      if (kmax16 - (int)t.key[f] != vk_idx) continue;
      const uint32_t tok = t.tok[f];
      uint32_t rank = 0;
#pragma unroll 1
      for (int j = 0; j < nties; ++j) rank += tie_tok[j] < tok ? 1u : 0u;
      if (rank >= (uint32_t)admitted) t.tok[f] = tok | 0x80000000u;
    }
    // each thread reads back only entries that it marked itself (same f stride below)
  }
  TLX_STAMP(sp, 10);
  // ---- Gumbel arg-max over the kept candidates, screened in f32 (four loads in flight per thread)
  const float inv_T = 1.0f / T_;
  const int kmin16 = kmax16 - vstar_idx;   // kept: key >= kmin16 and not marked
  float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
  int f1 = -1, t1 = 0x7FFFFFFF;
#pragma unroll 1
  for (int f0 = threadIdx.x; f0 < m; f0 += 4 * kStThreads) {
    float uu[4];
    uint32_t tk[4];
    int ky[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int f = f0 + u * kStThreads;
      tk[u] = f < m ? t.tok[f] : 0x80000000u;
      ky[u] = f < m ? (int)t.key[f] : 0;
      if (ky[u] < kmin16) tk[u] = 0x80000000u;
      uu[u] = (tk[u] >> 31) ? 0.5f : sp.noise.at(nrow, (int64_t)tk[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!(tk[u] >> 31)) {
        const float a = fmaf(key16_value(ky[u]), inv_T, gumbel_screen(uu[u]));
        const int tok = (int)tk[u];
        if (a > a1 || (a == a1 && tok < t1)) { a2 = a1; a1 = a; u1 = uu[u]; f1 = f0 + u * kStThreads; t1 = tok; }
        else if (a > a2) a2 = a;
      }
    }
  }
  TLX_STAMP(sp, 6);
  uint32_t bkey;
  int btok;
  tl_block_top(a1, t1, t, bkey, btok);
  const float amax = key_f32(bkey);
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  const bool mine = f1 >= 0 && f32_key(a1) == bkey && t1 == btok;
  const int multi = __syncthreads_or((f1 >= 0 && !mine && a1 >= cut) || a2 >= cut);
  TLX_STAMP(sp, 7);
  if (!multi) return btok;   // nothing else comes within the slack of the best screened score
  // several contenders: decide on the f64-evaluated Gumbel term
  const int crowded = __syncthreads_or(a2 >= cut);
  Best best{-INFINITY, 0x7FFFFFFF};
  if (!crowded) {
    if (f1 >= 0 && a1 >= cut) best = Best{__fdiv_rn(key16_value(t.key[f1]), T_) + gumbel_exact(u1), t1};
  } else {
#pragma unroll 1
    for (int f = threadIdx.x; f < m; f += kStThreads) {
      const uint32_t tok = t.tok[f];
      if ((int)t.key[f] >= kmin16 && !(tok >> 31)) {
        const float u = sp.noise.at(nrow, (int64_t)tok);
        const float x = key16_value(t.key[f]);
        if (fmaf(x, inv_T, gumbel_screen(u)) >= cut) best = best_of(best, Best{__fdiv_rn(x, T_) + gumbel_exact(u), (int)tok});
      }
    }
  }
  tl_block_top(best.y, best.tok, t, bkey, btok);
  return btok;
}

// One row of the finish kernel's row CTAs: normal rows are finished from their candidate lists; what that
// cannot settle takes the whole-row routines.
static __device__ __forceinline__ void st_finish_row(const StreamParams& p, int row, unsigned char* smem);

// A row that the short paths left unanswered: exact whole-row routines (out of line: rare and slow, and
// its stack frame and register needs stay out of the callers' way).  All threads call.
static __device__ __noinline__ void st_slow_row(const StreamParams& p, int row, unsigned char* smem) {
#ifdef TLX_SIZE_PROBE
  return;
#endif
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem + kSharedHeader);
  uint32_t* win = reinterpret_cast<uint32_t*>(smem + kSharedHeader);
  const SampleParams& sp = p.sp;
  const StreamDesc d = p.desc[row];
  const int64_t n = sp.vocab;
  const __nv_bfloat16* rowp = reinterpret_cast<const __nv_bfloat16*>(sp.logits) + (int64_t)row * sp.row_stride;
  const float pp = sp.top_p[row], T_ = sp.temperature[row];
  const int64_t nrow = row + sp.dim0_offset;
  int status = 0, tok = 0;
  __syncthreads();
  if (d.cls == kStNormal) {
    const int K = d.K;
    status = kStatusRedone;
    exact_select_row<TLX_BF16>(rowp, n, K, s, cand);
    __syncthreads();
    if (T_ < kSamplingEps) {
      uint64_t best = 0;
      for (int i = threadIdx.x; i < K; i += blockDim.x) {
        const uint64_t c = ~cand[i];
        best = c > best ? c : best;
      }
      block_max_u64(best, s);
      tok = (int)cand_low(~best);
    } else {
      tok = tail_bf16_hist(sp, row, K, pp, T_, K, s, cand);
      if (tok < 0) {
        __syncthreads();
        sort_candidates(cand, K);
        tok = sample_tail<4>(
            K, pp, T_, s, [&](int i) { return key_f32(cand_key(cand[i])); }, [&](int i) { return (int)cand_low(cand[i]); },
            [&](int i) { return sp.noise.at(nrow, (int64_t)cand_low(cand[i])); });
      }
    }
  } else {
    status = kStatusGeneral | (d.cls == kStWide ? (int)kStatusRedone : 0);
    int K = sp.top_k[row];
    if (K <= 0 || (int64_t)K >= n) K = (int)n;
    if (T_ < kSamplingEps) K = 1;
    if ((int64_t)K >= n && pp >= 1.0f) {
      tok = final_argmax<TLX_BF16>(rowp, n, T_, 0u, false, 0u, 0u, false, sp.noise, nrow, s);
    } else {
      RowPreset none;
      tok = general_row_bf16<kWin>(rowp, n, K, pp, T_, sp.noise, nrow, s, win, none);
    }
  }
  if (threadIdx.x == 0) {
    if (__ldcg(p.error_flag)) status |= kStatusTimeout;
    sp.out_tokens[row] = tok;
    if (sp.out_status) sp.out_status[row] = status;
  }
}

// ---- finish: final pass over the wide rows ------------------------------------------------------------
// One CTA per (wide row, range of the row's 8 KB chunks); the ranges are as short as the number of
// final-pass CTAs allows, so that the pass is a single wave.  A CTA keeps, per thread, the two best
// screened scores of its range and leaves ONE record: its best element, and whether anything else of the
// range comes within the screening slack of it.
constexpr size_t kFinSlotBytes = (size_t)kFinChunk + kFinNoiseChunk;
constexpr size_t kFinFixedSmem = kFinSlots * kFinSlotBytes + sizeof(StControl);   // + one int per row (the list)

__device__ __forceinline__ void fin_issue(const StreamParams& p, int row, int c, int c_end, bool dense,
                                          unsigned char* ring, unsigned long long* mbar, int slot) {
  if (c >= c_end) return;
  const int64_t off = (int64_t)c * kFinChunk;
  const int64_t rest = p.row_bytes - off;
  const uint32_t bytes = (uint32_t)(rest < kFinChunk ? rest : kFinChunk);
  unsigned char* dst = ring + (size_t)slot * kFinSlotBytes;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(p.sp.logits) + (int64_t)row * p.sp.row_stride * 2 + off;
  mbar_expect_tx(&mbar[slot], dense ? bytes * 3 : bytes);
  bulk_load(dst, src, bytes, &mbar[slot]);
  if (dense) {
    const float* nsrc = p.sp.noise.dense_row(row + p.sp.dim0_offset) + (int64_t)c * kFinChunkElems;
    bulk_load(dst + kFinChunk, nsrc, bytes * 2, &mbar[slot]);
  }
}

// Decides a wide row from the records of its ranges (all threads of the CTA that delivered the last one;
// at most kStThreads records).
// range_elems > 0: record i covers the elements [i * range_elems, (i + 1) * range_elems); 0: the final
// pass's ranges of chunks.
__device__ __forceinline__ void fin_decide_row(const StreamParams& p, int row, int nrec, int range_elems, StControl& ctl) {
  const SampleParams& sp = p.sp;
  const FinRecord* recs = p.records + (size_t)row * p.nfin;
  const float T_ = sp.temperature[row];
  const float inv_T = 1.0f / T_;
  const int64_t nrow = row + sp.dim0_offset;
  const int lane = lane_id(), warp = warp_id();
  // every thread takes one record; the best screened score over the row
  int4 r = make_int4(0, 0, 0x7FFFFFFF, 0);
  if ((int)threadIdx.x < nrec) r = __ldcg(reinterpret_cast<const int4*>(recs + threadIdx.x));
  const float a = __int_as_float(r.x), u = __int_as_float(r.y);
  const int tok = r.z;
  const uint32_t bits = (uint32_t)r.w;
  float amax = tok != 0x7FFFFFFF ? a : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  __syncthreads();
  if (lane == 0) ctl.fbest[warp] = amax;
  __syncthreads();
  amax = ctl.fbest[0];
#pragma unroll
  for (int w = 1; w < kStWarps; ++w) amax = fmaxf(amax, ctl.fbest[w]);
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  const bool contender = tok != 0x7FFFFFFF && a >= cut;
  Best best{-INFINITY, 0x7FFFFFFF};
  if (contender && !(bits & 0x10000u)) best = Best{__fdiv_rn(__uint_as_float(bits << 16), T_) + gumbel_exact(u), tok};
  // ranges in which several elements are close to the best: look at them again, one after the other (rare)
  uint32_t again = __ballot_sync(0xFFFFFFFFu, contender && (bits & 0x10000u));
  __syncthreads();
  if (lane == 0) ctl.wkey[warp] = again;
  __syncthreads();
  const uint32_t vstar16 = (uint32_t)wide_vstar16(__ldcg(&p.wstate[row].result));
  const float tvf = __uint_as_float(key16_bf16_bits(vstar16) << 16);
  const __nv_bfloat16* rowp = reinterpret_cast<const __nv_bfloat16*>(sp.logits) + (int64_t)row * sp.row_stride;
  for (int w = 0; w < kStWarps; ++w) {
    uint32_t mask = ctl.wkey[w];
    while (mask) {
      const int i = w * 32 + __ffs(mask) - 1;
      mask &= mask - 1;
      const int64_t e0 = range_elems > 0 ? (int64_t)i * range_elems : (int64_t)((int64_t)i * p.nfin / nrec) * kFinChunkElems;
      int64_t e1 = range_elems > 0 ? e0 + range_elems : (int64_t)((int64_t)(i + 1) * p.nfin / nrec) * kFinChunkElems;
      e1 = e1 < sp.vocab ? e1 : sp.vocab;
      for (int64_t c = e0 + threadIdx.x; c < e1; c += kStThreads) {
        const uint32_t b = *reinterpret_cast<const unsigned short*>(rowp + c);
        const float x = __uint_as_float(b << 16);
        if (!(x < tvf)) {
          const float un = sp.noise.at(nrow, c);
          if (fmaf(x, inv_T, gumbel_screen(un)) >= cut) best = best_of(best, Best{__fdiv_rn(x, T_) + gumbel_exact(un), (int)c});
        }
      }
    }
  }
  best = warp_best(best);
  __syncthreads();
  if (lane == 0) { ctl.fbest[warp] = best.y; ctl.ibest[warp] = best.tok; }
  __syncthreads();
  if (threadIdx.x == 0) {
    Best b{-INFINITY, 0x7FFFFFFF};
    for (int w = 0; w < kStWarps; ++w) b = best_of(b, Best{ctl.fbest[w], ctl.ibest[w]});
    sp.out_tokens[row] = b.tok == 0x7FFFFFFF ? 0 : b.tok;
  }
}

// The final-pass CTAs of the finish kernel (block indices below p.fin_ctas).
// dense != 0: the noise is a tensor whose rows can be bulk-copied (16-byte aligned); it is streamed next
// to the logits.  Otherwise the noise of the kept elements is read (or generated from the key) one by one.
static __device__ __forceinline__ void st_final_pass(const StreamParams& p, int dense, unsigned char* smem) {
#ifdef TLX_SIZE_PROBE2
  return;
#endif
  unsigned char* ring = smem;
  StControl& ctl = *reinterpret_cast<StControl*>(smem + kFinSlots * kFinSlotBytes);
  int* wlist = reinterpret_cast<int*>(smem + kFinFixedSmem);
  const SampleParams& sp = p.sp;
  const int lane = lane_id(), warp = warp_id();
  TLX_STAMP(sp, 0);
  if (threadIdx.x == 0) { ctl.cnt = 0; ctl.flag = 0; }
  asm volatile("griddepcontrol.wait;" ::: "memory");   // the wide rows' thresholds are in place
  __syncthreads();
  // the wide rows, in row order (every CTA builds the same list from the descriptors)
  for (int base = 0; base < (int)sp.rows; base += kStThreads) {
    const int r = base + (int)threadIdx.x;
    const bool wide = r < (int)sp.rows && p.desc[r].cls == kStWide;
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, wide);
    if (lane == 0) ctl.ibest[warp] = __popc(mask);
    __syncthreads();
    int off = ctl.cnt, total = 0;
    for (int w = 0; w < kStWarps; ++w) {
      if (w < warp) off += ctl.ibest[w];
      total += ctl.ibest[w];
    }
    if (wide) wlist[off + __popc(mask & ((1u << lane) - 1u))] = r;
    __syncthreads();
    if (threadIdx.x == 0) ctl.cnt += total;
    __syncthreads();
  }
  const int nwide = ctl.cnt;
  TLX_STAMP(sp, 1);
  if (nwide == 0) return;
  int J = p.fin_ctas / nwide;   // ranges per row
  J = J < 1 ? 1 : (J > p.nfin ? p.nfin : J);
  J = J > kStThreads ? kStThreads : J;
  // more wide rows than CTAs: a CTA takes several rows, one after the other
  for (int unit = blockIdx.x; unit < nwide * J; unit += p.fin_ctas) {
    const int w = unit / J, j = unit - w * J;
    const int row = wlist[w];
    WideState* ws = p.wstate + row;
    const int wres = __ldcg(&ws->result);
    const int vstar = wide_vstar16(wres);
    if (vstar < 0) continue;   // the row's own CTA answers it with the whole-row routines
    const int c_begin = (int)((int64_t)j * p.nfin / J), c_end = (int)((int64_t)(j + 1) * p.nfin / J);
    const uint32_t tbits = key16_bf16_bits((uint32_t)vstar);
    const __nv_bfloat162 tv2 = bf162_splat_bits(tbits);
    const float tvf = __uint_as_float(tbits << 16);
    const float T_ = sp.temperature[row];
    const float inv_T = 1.0f / T_;
    const int64_t nrow = row + sp.dim0_offset;
    const int last_nvec = (int)((p.row_bytes - (int64_t)(p.nfin - 1) * kFinChunk) >> 4);
    __syncthreads();   // the ring is idle (a previous unit has been consumed entirely)
    if (threadIdx.x == 0) {
      for (int s = 0; s < kFinSlots; ++s) mbar_init(&ctl.mbar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      ctl.best_key = f32_key(-INFINITY);
      for (int s = 0; s < kFinSlots; ++s) fin_issue(p, row, c_begin + s, c_end, dense != 0, ring, ctl.mbar, s);
    }
    __syncthreads();
    float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
    uint32_t b1 = 0;
    int t1 = 0x7FFFFFFF;
    int slot = 0;
    uint32_t phase = 0;
    // No element scores above (value of the row's maximum) / T + its own Gumbel term: once the CTA knows a
    // score `cb`, an element whose noise u gives -log(-log u) < cb - xtop - margin cannot come within the
    // screening slack of the best, and -log u <= 1 - u ... so the test is one comparison of 1 - u with
    // eps = exp(-(cb - xtop - margin)) (1 - u >= 1 - exp(-eps') for the exact bound eps'; eps is looser).
    const float xtop = key16_value(wide_kmax16(wres)) * inv_T;
    float published = -INFINITY;
    for (int c = c_begin; c < c_end; ++c) {
      const float cb = key_f32(ctl.best_key);
      const float eps = expf(-(cb - 2.0f * (kGumbelSlack + 1e-5f * fabsf(cb)) - xtop)) * 1.000001f;
      const bool arrived = mbar_wait_suspended(&ctl.mbar[slot], phase);
      if (c == c_begin && unit == (int)blockIdx.x) TLX_STAMP(sp, 2);
      const unsigned char* buf = ring + (size_t)slot * kFinSlotBytes;
      const float* nbuf = reinterpret_cast<const float*>(buf + kFinChunk);
      const int nvec = (c == p.nfin - 1) ? last_nvec : kFinChunk / 16;
      if (!(p.debug & 2)) {
#pragma unroll 1
        for (int jv = 0; jv < kFinVecPerThread; ++jv) {
          const int v = (int)threadIdx.x + jv * kStThreads;
          if (v < nvec) {
            const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
            const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(x.x), bf162_bits(x.y)),
                                                 __hmax2_nan(bf162_bits(x.z), bf162_bits(x.w)));
            if (!__hblt2(m, tv2)) {
              // eight independent screened scores, then their best two
              const uint32_t wd[4] = {x.x, x.y, x.z, x.w};
              float un[8];
              if (dense) {
                const float4 n0 = *reinterpret_cast<const float4*>(nbuf + v * 8);
                const float4 n1 = *reinterpret_cast<const float4*>(nbuf + v * 8 + 4);
                un[0] = n0.x; un[1] = n0.y; un[2] = n0.z; un[3] = n0.w;
                un[4] = n1.x; un[5] = n1.y; un[6] = n1.z; un[7] = n1.w;
                const float umax = fmaxf(fmaxf(fmaxf(un[0], un[1]), fmaxf(un[2], un[3])),
                                         fmaxf(fmaxf(un[4], un[5]), fmaxf(un[6], un[7])));
                if (1.0f - umax > eps) continue;   // none of the eight can matter
              }
              float sc[8];
              float v1 = -INFINITY, v2 = -INFINITY;
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const uint32_t hi = (e & 1) ? (wd[e >> 1] & 0xFFFF0000u) : (wd[e >> 1] << 16);
                const float xf = __uint_as_float(hi);
                bool keep = !(xf < tvf);
                if (!dense) un[e] = keep ? sp.noise.at(nrow, c * kFinChunkElems + v * 8 + e) : 0.5f;
                keep = keep && 1.0f - un[e] <= eps;
                sc[e] = keep ? fmaf(xf, inv_T, gumbel_screen(un[e])) : -INFINITY;
                const float lo = fminf(v1, sc[e]);
                v1 = fmaxf(v1, sc[e]);
                v2 = fmaxf(v2, lo);
              }
              if (v1 > a1) {
                int ebest = 0;
#pragma unroll
                for (int e = 7; e >= 0; --e) if (sc[e] == v1) ebest = e;
                u1 = un[0];
                b1 = wd[0] & 0xFFFFu;
#pragma unroll
                for (int e = 1; e < 8; ++e)
                  if (e == ebest) { u1 = un[e]; b1 = (e & 1) ? (wd[e >> 1] >> 16) : (wd[e >> 1] & 0xFFFFu); }
                t1 = c * kFinChunkElems + v * 8 + ebest;
              }
              a2 = fmaxf(fminf(a1, v1), fmaxf(a2, v2));
              a1 = fmaxf(a1, v1);
            }
          }
        }
      }
      if (a1 > published) { atomicMax(&ctl.best_key, f32_key(a1)); published = a1; }
      if (__syncthreads_or(!arrived)) {   // a copy never arrived: give up, the row's status says so
        if (threadIdx.x == 0 && sp.out_status) atomicOr(sp.out_status + row, (int)kStatusTimeout);
        return;
      }
      if (threadIdx.x == 0) fin_issue(p, row, c + kFinSlots, c_end, dense != 0, ring, ctl.mbar, slot);
      if (++slot == kFinSlots) { slot = 0; phase ^= 1u; }
    }
    if (unit == (int)blockIdx.x) TLX_STAMP(sp, 3);
    if (p.debug & 4) continue;
    // the range's record
    const uint32_t key = f32_key(a1);
    const uint32_t wkey = __reduce_max_sync(0xFFFFFFFFu, key);
    const int wtok = __reduce_min_sync(0xFFFFFFFFu, key == wkey ? t1 : 0x7FFFFFFF);
    if (lane == 0) { ctl.wkey[warp] = wkey; ctl.wtok[warp] = wtok; }
    __syncthreads();
    uint32_t bkey = ctl.wkey[0];
    int btok = ctl.wtok[0];
#pragma unroll
    for (int i = 1; i < kStWarps; ++i) {
      const uint32_t k = ctl.wkey[i];
      const int tk = ctl.wtok[i];
      if (k > bkey || (k == bkey && tk < btok)) { bkey = k; btok = tk; }
    }
    const bool any = btok != 0x7FFFFFFF;
    const bool mine = any ? (key == bkey && t1 == btok) : threadIdx.x == 0;
    const float amax = key_f32(bkey);
    const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
    const int multi = __syncthreads_or(any && ((!mine && a1 >= cut) || a2 >= cut));
    if (mine) {
      FinRecord r;
      r.a = a1; r.u = u1; r.tok = any ? t1 : 0x7FFFFFFF; r.bits = b1 | (multi ? 0x10000u : 0u);
      p.records[(size_t)row * p.nfin + j] = r;
      __threadfence();
      ctl.flag = (atomicAdd(&ws->done, 1) == J - 1) ? 1 : 0;
    }
    __syncthreads();
    if (unit == (int)blockIdx.x) TLX_STAMP(sp, 4);
    if (ctl.flag) {
      __threadfence();
      TLX_STAMP(sp, 6);
      fin_decide_row(p, row, J, 0, ctl);
      TLX_STAMP(sp, 7);
    }
  }
  TLX_STAMP(sp, 5);
}

static __device__ __forceinline__ void st_finish_row(const StreamParams& p, int row, unsigned char* smem) {
  TailShared& t = *reinterpret_cast<TailShared*>(smem);
  const SampleParams& sp = p.sp;
  for (int i = threadIdx.x; i < kTlBins; i += kStThreads) t.hist[i] = 0;
  // This CTA started after the prologue kernel had completed (see the stream kernel): the row's descriptor is
  // there.  It waits for its own row only: a normal row's P parts, a wide row's final items; the stream kernel
  // may go on with other rows meanwhile.  The waits are bounded; past the bound (and for rows that the
  // whole-row routines take) the CTA waits for the whole stream kernel.
  static_assert(sizeof(StreamDesc) == 16, "StreamDesc is read as one 16-byte word");
  const uint4 draw = __ldcg(reinterpret_cast<const uint4*>(p.desc + row));
  StreamDesc d;
  memcpy(&d, &draw, sizeof(d));
  if (threadIdx.x == 0) {
    volatile const int* flag = nullptr;
    int want = 0;
    const bool signals = *reinterpret_cast<volatile const int*>(p.row_signals) != 0;
    if (d.cls == kStNormal && signals) { flag = p.rowdone + row; want = p.P; }
    else if (d.cls == kStWide && p.fin_items > 0) { flag = &p.wstate[row].done; want = p.fin_items; }
    bool ready = false;
    if (flag && !(p.debug & 16)) {
      for (int spin = 0; spin < (1 << 18) && !(ready = *flag >= want); ++spin) __nanosleep(100);
    }
    if (!ready) asm volatile("griddepcontrol.wait;" ::: "memory");
    __threadfence();
  }
  __syncthreads();
  // one round trip for everything the row's short path reads first (whatever the row's class turns out to be)
  const float pp = sp.top_p[row], T_ = sp.temperature[row];
  const int timeout = __ldcg(p.error_flag) ? (int)kStatusTimeout : 0;
  const TailFetch fetched = tl_fetch(p, row);
  TLX_STAMP(sp, 0);
  __syncthreads();
  bool slow = d.cls == kStOther;
  if (d.cls == kStNormal) {
    TLX_STAMP(sp, 1);
    const int tok = st_finish_normal(p, row, d, pp, T_, fetched, t);
    slow = tok < 0;   // threshold too high for this row, a list overflowed, or keys too far apart
    if (!slow && threadIdx.x == 0) {
      sp.out_tokens[row] = tok;
      if (sp.out_status) sp.out_status[row] = timeout;
    }
  } else if (d.cls == kStWide) {
    // the window did not settle the threshold, or (final items in the stream kernel) something went wrong there
    slow = __ldcg(&p.wstate[row].result) < 0 || (p.fin_items > 0 && timeout);
    if (!slow && p.fin_items > 0) {
      // the stream kernel has left a record per final item of the row: decide
      StControl& ctl = *reinterpret_cast<StControl*>(smem + kFinSlots * kFinSlotBytes);
      __syncthreads();
      fin_decide_row(p, row, p.fin_items, kStFinalElems, ctl);
    }
    if (!slow && threadIdx.x == 0 && sp.out_status) atomicOr(sp.out_status + row, (int)kStatusGeneral | timeout);
  }
  TLX_STAMP(sp, 8);
  if (threadIdx.x == 0 && sp.timeline) sp.timeline[(size_t)blockIdx.x * 16 + 9] = d.cls;
  if (slow) st_slow_row(p, row, smem);
  // this kernel must not be complete before the stream kernel is: whatever follows on the stream may reuse
  // the workspace
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

constexpr size_t kStFinishRowSmem =
    sizeof(TailShared) > kSharedHeader + kUnionBytes ? sizeof(TailShared) : kSharedHeader + kUnionBytes;
constexpr size_t kStFinishFixedSmem =
    kStFinishRowSmem > kFinFixedSmem ? kStFinishRowSmem : kFinFixedSmem;   // + one int per row (the final pass's list)

// Grid: p.fin_ctas CTAs of the final pass, then one CTA per row.
__global__ void __launch_bounds__(kStThreads, 3) sample_finish_kernel(StreamParams p, int dense) {
  extern __shared__ __align__(128) unsigned char fin_smem[];
  if ((int)blockIdx.x < p.fin_ctas) st_final_pass(p, dense, fin_smem);
  else st_finish_row(p, (int)blockIdx.x - p.fin_ctas, fin_smem);
}

}  // namespace tlx
