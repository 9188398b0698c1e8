// Row-per-CTA form of the fused sampler for bf16 logits whose rows start on 16-byte boundaries, for
// batches with at least about one row per SM.  Included by sampler.cu after sampler_stream.cuh (whose
// bit helpers, row classes and wide-row threshold search it shares).
//
// One kernel, no workspace, no communication between CTAs.  A CTA (512 threads, two per SM) owns a row at a time
// and streams it through a ring of four 16 KB bulk copies (cp.async.bulk + mbarrier) in shared memory, so that
// an SM keeps 128 KB in flight:
//   start      the ring's first copies are requested at once (the chunks are visited in a strided order, so
//              these are spread over the row); a 4096-element sample out of them and the row's parameters
//              give the row's class and
//                normal (1 <= top_k <= 1024, or greedy): the 16-bit key threshold that, with four
//                    standard deviations of margin, keeps at least top_k elements of the row;
//                wide   (top-k disabled, top_p < 1): the top of the histogram window, 512 keys above the
//                    sample's maximum;
//                plain  (top-k disabled, top_p >= 1): nothing, every element is kept;
//                other  (a larger top_k): the whole-row routines of sampler_general.cuh.
//   normal     pass over the row: one packed compare per 16-byte vector, the warp notes the vectors that
//              hold something, looks at them densely (one element per lane) and appends (token, bits) to
//              its own list in shared memory.  Tail: one histogram over the candidates' keys gives the
//              top-k boundary, the softmax mass over the top-k set and the top-p threshold (the mass of a
//              value group is count * exp(value - max)); the kept candidates' noise is the only thing
//              fetched from global memory; Gumbel arg-max, screened in f32 and decided on the
//              f64-evaluated term when several candidates come within the screening slack.
//   wide       pass over the row: histogram of the 16-bit keys inside the window, sum of exp(x - window
//              top) below it; row maximum, denominator and top-p threshold key from them.  If at most
//              4096 elements are kept: second pass (the row now comes from L2) with the candidate filter
//              at the threshold, then the normal rows' scoring over everything collected.  Otherwise,
//              and for plain rows: a pass with the logits and their noise streamed side by side, two best
//              screened scores per thread.
// A row whose threshold was too high, whose lists overflowed or whose window did not settle it takes the
// exact whole-row routines.
#pragma once

namespace tlx {

constexpr int kRwThreads = 256;
constexpr int kRwWarps = kRwThreads / 32;
constexpr int kRwChunk = 16384;                       // bytes per bulk copy and ring slot
constexpr int kRwChunkElems = kRwChunk / 2;
constexpr int kRwChunkVecs = kRwChunk / 16;
constexpr int kRwVecPerThread = kRwChunkVecs / kRwThreads;   // 2
constexpr int kRwSlots = 4;
constexpr int kRwWarpCap = 512;                       // candidates per warp and row
constexpr int kRwCap = kRwWarpCap * kRwWarps;         // 4096
constexpr int kRwBins = kStWin;                       // histogram bins: a wide row's window, or keys above a normal row's threshold
constexpr int kRwKeys = kStSample / kRwThreads;          // sample keys per thread
constexpr int kRwSelBins = 2048;                      // threshold selection: keys below the sample's maximum that are told apart
constexpr int kRwDenseElems = 4096;                   // dense pass: elements per group (8 KB of logits + 16 KB of noise)
constexpr int kRwDenseGroups = 2;
static_assert(kRwBins % kRwThreads == 0 && kRwSelBins % kRwThreads == 0, "bins per thread");
static_assert(kRwSelBins * 4 <= kRwCap * 4, "the selection histogram lives in the token lists");
static_assert(kRwDenseGroups * kRwDenseElems * 6 <= kRwSlots * kRwChunk, "the dense pass's groups fit the ring");

enum RwClass : int { kRwNormal = 0, kRwWide = 1, kRwPlain = 2, kRwOther = 3 };

struct RowsParams {
  SampleParams sp;
  int nchunks;           // 16 KB chunks per row (the last one may be short)
  int last_nvec;         // 16-byte vectors of the last chunk
  int stride;            // the chunks are visited in the order 0, stride, 2 stride, ... (mod nchunks; coprime)
  int64_t row_bytes;
  int dense_noise;       // the noise is a tensor whose rows can be bulk-copied
  int debug;
};

struct __align__(16) RwControl {
  unsigned long long mbar[kRwSlots];
  int red[kRwWarps];
  int sel_key, sel_pad;
  int wcnt[kRwWarps];
  uint32_t scan_c[kRwWarps];
  double scan_m[kRwWarps];
  double Z;
  int maxbin, overflow, nties, timeout;
  int vk_idx, admitted, ties_total, vstar_idx;
  uint32_t wkey[kRwWarps];
  int wtok[kRwWarps];
  float fbest[kRwWarps];
  int ibest[kRwWarps];
  WideScratch wide;
};

// Shared memory: ring | hist | tok | bits | vector lists | control.  The whole-row routines' scratch overlays
// the ring.
struct RwSmem {
  unsigned char* ring;
  uint32_t* hist;          // kRwBins
  uint32_t* tok;           // kRwCap, warp w owns [w * kRwWarpCap, (w + 1) * kRwWarpCap)
  unsigned short* bits;    // kRwCap
  unsigned short* vlist;   // per warp 32 * kRwVecPerThread vector indices
  RwControl* ctl;
};
constexpr size_t kRwListBytes = (size_t)kRwWarps * 32 * kRwVecPerThread * 2;
constexpr size_t kRwRingBytes = (size_t)kRwSlots * kRwChunk;
constexpr size_t kRwSmemBytes = kRwRingBytes + (size_t)kRwBins * 4 + (size_t)kRwCap * 4 + (size_t)kRwCap * 2 + kRwListBytes +
                                sizeof(RwControl);
static_assert(kRwRingBytes >= kSharedHeader + kUnionBytes, "the whole-row routines' scratch overlays the ring");

// Waits for the copies requested at a row's start without using them (the row takes another route).
__device__ __forceinline__ bool rw_drain(const RowsParams& p, RwSmem& sm, uint32_t& phases) {
  bool ok = true;
  const int n = p.nchunks < kRwSlots ? p.nchunks : kRwSlots;
  for (int sl = 0; sl < n; ++sl) {
    ok &= mbar_wait_suspended(&sm.ctl->mbar[sl], (phases >> sl) & 1u);
    phases ^= 1u << sl;
  }
  return !__syncthreads_or(!ok);
}

// The i-th chunk visited is chunk (i * stride) mod nchunks: the first copies of a row are spread over it,
// so that they can serve as the sample for the threshold.
__device__ __forceinline__ int rw_chunk_of(const RowsParams& p, int i) { return (int)(((int64_t)i * p.stride) % p.nchunks); }

__device__ __forceinline__ void rw_issue(const RowsParams& p, const unsigned char* rowp, int i, RwSmem& sm, int slot) {
  if (i >= p.nchunks) return;
  const int c = rw_chunk_of(p, i);
  const int64_t off = (int64_t)c * kRwChunk;
  const int64_t rest = p.row_bytes - off;
  const uint32_t bytes = (uint32_t)(rest < kRwChunk ? rest : kRwChunk);
  mbar_expect_tx(&sm.ctl->mbar[slot], bytes);
  bulk_load(sm.ring + (size_t)slot * kRwChunk, rowp + off, bytes, &sm.ctl->mbar[slot]);
}

// One pass over the row's chunks through the ring: f(buf, nvec, chunk, full) for every chunk, in visiting
// order.  `phases` holds the slots' mbarrier phases (it lives across passes).  If `primed`, the pass's
// first `slots` copies have been requested already.  Returns false if a copy did not arrive (bounded wait).
template <typename F>
__device__ __forceinline__ bool rw_pass(const RowsParams& p, const unsigned char* rowp, RwSmem& sm, uint32_t& phases,
                                        bool primed, F&& f) {
  if (!primed && threadIdx.x == 0)
    for (int s = 0; s < kRwSlots; ++s) rw_issue(p, rowp, s, sm, s);
  int slot = 0, c = 0;
  for (int i = 0; i < p.nchunks; ++i) {
    const bool arrived = mbar_wait_suspended(&sm.ctl->mbar[slot], (phases >> slot) & 1u);
    phases ^= 1u << slot;
    const bool full = c != p.nchunks - 1;
    f(sm.ring + (size_t)slot * kRwChunk, full ? kRwChunkVecs : p.last_nvec, c, full);
    if (__syncthreads_or(!arrived)) return false;
    if (threadIdx.x == 0) rw_issue(p, rowp, i + kRwSlots, sm, slot);   // the chunk is consumed, its slot is free
    if (++slot == kRwSlots) slot = 0;
    c += p.stride;
    if (c >= p.nchunks) c -= p.nchunks;
  }
  return true;
}

// The r-th largest of the kRwKeys keys each thread holds (4096 in all): a histogram of the keys in the
// kRwSelBins-key window below the sample's maximum (`bins`: that many words of shared memory, any
// contents), scanned from the top.  If fewer than r keys lie in the window, its lowest key is returned
// (a threshold that is lower than asked for).  r in [1, 4096].  All threads call.
__device__ __forceinline__ int rw_select_key(const uint32_t (&key)[kRwKeys], int r, uint32_t* bins, RwControl& ctl) {
  constexpr int kPer = kRwSelBins / kRwThreads;   // 4
  const int lane = lane_id(), warp = warp_id();
  uint32_t m = key[0];
#pragma unroll
  for (int i = 1; i < kRwKeys; ++i) m = max(m, key[i]);
  m = __reduce_max_sync(0xFFFFFFFFu, m);
  if (lane == 0) ctl.red[warp] = (int)m;
#pragma unroll
  for (int j = 0; j < kPer; ++j) bins[threadIdx.x + j * kRwThreads] = 0;
  __syncthreads();
  int top = ctl.red[0];
#pragma unroll
  for (int w = 1; w < kRwWarps; ++w) top = max(top, ctl.red[w]);
#pragma unroll
  for (int i = 0; i < kRwKeys; ++i) {
    const int d = top - (int)key[i];
    if (d < kRwSelBins) atomicAdd(&bins[d], 1u);
  }
  if (threadIdx.x == 0) ctl.sel_key = max(top - (kRwSelBins - 1), 0);
  __syncthreads();
  // thread t owns the bins [kPer t, kPer t + kPer): descending keys over the block
  uint32_t c[kPer];
  uint32_t local = 0;
#pragma unroll
  for (int j = 0; j < kPer; ++j) { c[j] = bins[threadIdx.x * kPer + j]; local += c[j]; }
  uint32_t incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) ctl.scan_c[warp] = incl;
  __syncthreads();
  for (int w = 0; w < warp; ++w) incl += ctl.scan_c[w];
  uint32_t run = incl - local;
  if (run < (uint32_t)r && incl >= (uint32_t)r) {
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (run < (uint32_t)r && run + c[j] >= (uint32_t)r) ctl.sel_key = top - ((int)threadIdx.x * kPer + j);
      run += c[j];
    }
  }
  __syncthreads();
  return ctl.sel_key;
}

// Candidate filter of one chunk: elements that are not below the threshold value (a NaN is one) go to the
// warp's list as (token, bf16 bits).  wl: the warp's list of vectors that may hold one.
template <bool kFull>
__device__ __forceinline__ void rw_filter_chunk(const unsigned char* buf, int nvec, int tok0, float tvf, __nv_bfloat162 tv2,
                                                uint32_t* wtok, unsigned short* wbits, int& wc, unsigned short* wl) {
  const int lane = lane_id();
  const uint32_t lt = (1u << lane) - 1u;
  int wn = 0;
#pragma unroll
  for (int j = 0; j < kRwVecPerThread; ++j) {
    const int v = (int)threadIdx.x + j * kRwThreads;
    bool hit = false;
    if (kFull || v < nvec) {
      const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
      const __nv_bfloat162 m =
          __hmax2_nan(__hmax2_nan(bf162_bits(x.x), bf162_bits(x.y)), __hmax2_nan(bf162_bits(x.z), bf162_bits(x.w)));
      hit = !__hblt2(m, tv2);
    }
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, hit);
    if (mask) {
      if (hit) wl[wn + __popc(mask & lt)] = (unsigned short)v;
      wn += __popc(mask);
    }
  }
  if (wn == 0) return;
  __syncwarp();
  for (int base = 0; base < wn; base += 4) {
    const int e = base + (lane >> 3);
    bool pass = false;
    uint32_t b = 0;
    int q = 0;
    if (e < wn) {
      q = wl[e] * 8 + (lane & 7);
      b = reinterpret_cast<const unsigned short*>(buf)[q];
      pass = !(__uint_as_float(b << 16) < tvf);
    }
    const uint32_t pm = __ballot_sync(0xFFFFFFFFu, pass);
    const int pos = wc + __popc(pm & lt);
    if (pass && pos < kRwWarpCap) { wtok[pos] = (uint32_t)(tok0 + q); wbits[pos] = (unsigned short)b; }
    wc += __popc(pm);
  }
  __syncwarp();
}

// Block-wide (max score, lowest token) over one candidate per thread; valid in every thread.
__device__ __forceinline__ void rw_block_top(float a, int tok, RwControl& ctl, uint32_t& bkey, int& btok) {
  const uint32_t key = f32_key(a);
  const uint32_t wkey = __reduce_max_sync(0xFFFFFFFFu, key);
  const int wtok = __reduce_min_sync(0xFFFFFFFFu, key == wkey ? tok : 0x7FFFFFFF);
  __syncthreads();
  if (lane_id() == 0) { ctl.wkey[warp_id()] = wkey; ctl.wtok[warp_id()] = wtok; }
  __syncthreads();
  bkey = ctl.wkey[0];
  btok = ctl.wtok[0];
#pragma unroll
  for (int i = 1; i < kRwWarps; ++i) {
    const uint32_t k = ctl.wkey[i];
    const int tk = ctl.wtok[i];
    if (k > bkey || (k == bkey && tk < btok)) { bkey = k; btok = tk; }
  }
}

// What decides whether a candidate of the lists is kept.
struct RwKeep {
  bool all;            // wide rows' second pass: everything collected is kept
  int kmax16, vstar_idx, vk_idx, admitted;
  bool cut_ties;
  int nties;
  const uint32_t* tie_tok;
  __device__ __forceinline__ bool operator()(uint32_t tok, uint32_t bits) const {
    if (all) return true;
    const int idx = kmax16 - (int)bf16_key16(bits);
    if (idx > vstar_idx) return false;
    if (idx < vk_idx || !cut_ties) return true;
    uint32_t rank = 0;
    for (int j = 0; j < nties; ++j) rank += tie_tok[j] < tok ? 1u : 0u;
    return rank < (uint32_t)admitted;
  }
};

// Gumbel arg-max over the kept candidates of the warps' lists (wc: this warp's count): screened in f32,
// decided on the f64-evaluated Gumbel term when several candidates come within the slack.  All threads call.
__device__ __forceinline__ int rw_score_lists(const SampleParams& sp, int64_t nrow, float T_, RwKeep keep,
                                                  RwSmem& sm, int wc) {
  const int lane = lane_id(), warp = warp_id();
  const uint32_t* wtok = sm.tok + warp * kRwWarpCap;
  const unsigned short* wbits = sm.bits + warp * kRwWarpCap;
  const float inv_T = 1.0f / T_;
  float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
  uint32_t b1 = 0;
  int t1 = 0x7FFFFFFF;
#pragma unroll 1
  for (int i0 = lane; i0 < wc; i0 += 8 * 32) {
    float uu[8];
    uint32_t kk = 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * 32;
      const bool k = i < wc && keep(wtok[i], wbits[i]);
      kk |= (k ? 1u : 0u) << u;
      uu[u] = k ? sp.noise.at(nrow, (int64_t)wtok[i]) : 0.5f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * 32;
      if (kk & (1u << u)) {
        const uint32_t b = wbits[i];
        const float a = fmaf(__uint_as_float(b << 16), inv_T, gumbel_screen(uu[u]));
        const int tk = (int)wtok[i];
        if (a > a1 || (a == a1 && tk < t1)) { a2 = a1; a1 = a; u1 = uu[u]; b1 = b; t1 = tk; }
        else if (a > a2) a2 = a;
      }
    }
  }
  RwControl& ctl = *sm.ctl;
  TLX_STAMP(sp, 12);
  uint32_t bkey;
  int btok;
  rw_block_top(a1, t1, ctl, bkey, btok);
  const float amax = key_f32(bkey);
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  const bool have = t1 != 0x7FFFFFFF;
  const bool mine = have && f32_key(a1) == bkey && t1 == btok;
  const int multi = __syncthreads_or((have && !mine && a1 >= cut) || a2 >= cut);
  TLX_STAMP(sp, 13);
  if (threadIdx.x == 0 && sp.timeline) sp.timeline[(size_t)blockIdx.x * 16 + 14] = multi * 1000000 + wc;
  if (!multi) return btok;   // nothing else comes within the slack of the best screened score
  const int crowded = __syncthreads_or(a2 >= cut);
  Best best{-INFINITY, 0x7FFFFFFF};
  if (!crowded) {
    if (have && a1 >= cut) best = Best{__fdiv_rn(__uint_as_float(b1 << 16), T_) + gumbel_exact(u1), t1};
  } else {
    for (int i = lane; i < wc; i += 32) {
      if (keep(wtok[i], wbits[i])) {
        const float u = sp.noise.at(nrow, (int64_t)wtok[i]);
        const float x = __uint_as_float((uint32_t)wbits[i] << 16);
        if (fmaf(x, inv_T, gumbel_screen(u)) >= cut) best = best_of(best, Best{__fdiv_rn(x, T_) + gumbel_exact(u), (int)wtok[i]});
      }
    }
  }
  rw_block_top(best.y, best.tok, ctl, bkey, btok);
  return btok;
}

// Tail of a normal row over the warps' candidate lists (all taken at or above the key thr16).  Returns
// the token, or -1 if the lists cannot be trusted to hold the row's top-K or the candidates' keys spread
// over more than kRwBins values.  hist[] must be zero.  All threads call.
__device__ __forceinline__ int rw_tail_normal(const SampleParams& sp, int64_t nrow, int K, int thr16, float pp, float T_,
                                                  RwSmem& sm, int wc) {
  RwControl& ctl = *sm.ctl;
  const int lane = lane_id(), warp = warp_id();
  const uint32_t* wtok = sm.tok + warp * kRwWarpCap;
  const unsigned short* wbits = sm.bits + warp * kRwWarpCap;
  if (lane == 0) ctl.wcnt[warp] = wc;
  if (threadIdx.x == 0) { ctl.maxbin = 0; ctl.overflow = 0; ctl.nties = 0; }
  __syncthreads();
  int m = 0, bad = 0;
#pragma unroll
  for (int w = 0; w < kRwWarps; ++w) { m += ctl.wcnt[w]; bad |= ctl.wcnt[w] > kRwWarpCap; }
  if (bad || m < K) return -1;
  // ---- greedy: the greatest key, lowest token
  if (T_ < kSamplingEps) {
    uint32_t bk = 0;
    int bt = 0x7FFFFFFF;
    for (int i = lane; i < wc; i += 32) {
      const uint32_t k = bf16_key16(wbits[i]);
      const int tk = (int)wtok[i];
      if (k > bk || (k == bk && tk < bt)) { bk = k; bt = tk; }
    }
    const uint32_t wk = __reduce_max_sync(0xFFFFFFFFu, bk);
    const int wt = __reduce_min_sync(0xFFFFFFFFu, bk == wk ? bt : 0x7FFFFFFF);
    if (lane == 0) { ctl.wkey[warp] = wk; ctl.wtok[warp] = wt; }
    __syncthreads();
    uint32_t k0 = ctl.wkey[0];
    int t0 = ctl.wtok[0];
    for (int i = 1; i < kRwWarps; ++i)
      if (ctl.wkey[i] > k0 || (ctl.wkey[i] == k0 && ctl.wtok[i] < t0)) { k0 = ctl.wkey[i]; t0 = ctl.wtok[i]; }
    return t0;
  }
  // ---- histogram over the candidates' keys
  {
    int mymax = 0, over = 0;
    for (int i = lane; i < wc; i += 32) {
      const int bin = (int)bf16_key16(wbits[i]) - thr16;
      if (bin >= 0 && bin < kRwBins) { atomicAdd(&sm.hist[bin], 1u); mymax = max(mymax, bin); }
      else over = 1;
    }
    mymax = __reduce_max_sync(0xFFFFFFFFu, mymax);
    if (lane == 0) atomicMax(&ctl.maxbin, mymax);
    if (over) ctl.overflow = 1;
  }
  __syncthreads();
  if (ctl.overflow) return -1;
  TLX_STAMP(sp, 10);
  // ---- one scan over the bins in descending key order: counts and (unbounded) mass
  const int maxbin = ctl.maxbin;
  const int W = maxbin + 1;
  const int kmax16 = thr16 + maxbin;
  const float xmax = key16_value(kmax16);
  const int per = (W + kRwThreads - 1) / kRwThreads;
  const int i0 = threadIdx.x * per;   // idx = maxbin - bin
  uint32_t lc = 0;
  double lm = 0.0;
#pragma unroll 1
  for (int j = 0; j < per; ++j) {
    const int idx = i0 + j;
    if (idx < W) {
      const uint32_t c = sm.hist[maxbin - idx];
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
  if (lane == 31) { ctl.scan_c[warp] = ic; ctl.scan_m[warp] = im; }
  __syncthreads();
  for (int w = 0; w < warp; ++w) { ic += ctl.scan_c[w]; im += ctl.scan_m[w]; }
  const uint32_t ec = ic - lc;   // exclusive prefixes
  const double em = im - lm;
  if (ec < (uint32_t)K && ic >= (uint32_t)K) {
    // the top-k boundary lies in this thread's bins
    uint32_t run = ec;
    double mass = em;
#pragma unroll 1
    for (int j = 0; j < per; ++j) {
      const int idx = i0 + j;
      const uint32_t c = sm.hist[maxbin - idx];
      const double ex = (double)expf(key16_value(kmax16 - idx) - xmax);
      if (run + c >= (uint32_t)K) {
        ctl.vk_idx = idx;
        ctl.admitted = (int)((uint32_t)K - run);
        ctl.ties_total = (int)c;
        ctl.Z = mass + (double)((uint32_t)K - run) * ex;
        ctl.vstar_idx = idx;   // default: the whole top-k set is kept
        break;
      }
      run += c;
      mass += (double)c * ex;
    }
  }
  __syncthreads();
  const int vk_idx = ctl.vk_idx, admitted = ctl.admitted, ties_total = ctl.ties_total;
  const double target = (double)pp * ctl.Z;
  if (em < target && i0 <= vk_idx) {
    // first value group at which the cumulative mass over the top-k set reaches top_p * Z
    double run = em;
#pragma unroll 1
    for (int j = 0; j < per; ++j) {
      const int idx = i0 + j;
      if (idx > vk_idx) break;
      const uint32_t c = idx == vk_idx ? (uint32_t)admitted : sm.hist[maxbin - idx];
      if (c) {
        run += (double)c * (double)expf(key16_value(kmax16 - idx) - xmax);
        if (run >= target) { ctl.vstar_idx = idx; break; }
      }
    }
  }
  __syncthreads();
  RwKeep keep;
  keep.all = false;
  keep.kmax16 = kmax16;
  keep.vstar_idx = ctl.vstar_idx;
  keep.vk_idx = vk_idx;
  keep.admitted = admitted;
  keep.cut_ties = keep.vstar_idx == vk_idx && admitted < ties_total;
  keep.tie_tok = sm.hist;   // the histogram is no longer needed
  // the lowest tokens of the boundary group are the admitted ones: list the group's tokens
  if (keep.cut_ties) {
    __syncthreads();
    for (int i = lane; i < wc; i += 32)
      if (kmax16 - (int)bf16_key16(wbits[i]) == vk_idx) sm.hist[atomicAdd(&ctl.nties, 1)] = wtok[i];
    __syncthreads();
  }
  keep.nties = ctl.nties;
  TLX_STAMP(sp, 11);
  return rw_score_lists(sp, nrow, T_, keep, sm, wc);
}

// Pass over a row with its noise streamed next to the logits (two groups in the ring, each 8 KB of logits
// followed by their 16 KB of noise): arg-max of x / T + gumbel(u) over the elements that are not below tvf
// (all of them if tvf is a NaN).  Needs p.dense_noise; the ring must be idle.  Returns the token; all
// threads call.
__device__ __forceinline__ int rw_dense_pass(const RowsParams& p, int64_t row, float T_, float tvf, __nv_bfloat162 tv2,
                                                 RwSmem& sm, uint32_t& phases, bool& ok) {
  constexpr int kGroupBytes = kRwDenseElems * 6;
  const SampleParams& sp = p.sp;
  RwControl& ctl = *sm.ctl;
  const unsigned char* rowp = reinterpret_cast<const unsigned char*>(sp.logits) + row * sp.row_stride * 2;
  const int64_t nrow = row + sp.dim0_offset;
  const float* nrowp = sp.noise.dense_row(nrow);
  const int ngroups = (int)((sp.vocab + kRwDenseElems - 1) / kRwDenseElems);
  const float inv_T = 1.0f / T_;
  auto issue = [&](int c, int g) {
    if (c >= ngroups) return;
    const int64_t e0 = (int64_t)c * kRwDenseElems;
    const int64_t rest = sp.vocab - e0;
    const uint32_t elems = (uint32_t)(rest < kRwDenseElems ? rest : kRwDenseElems);   // a multiple of 8
    unsigned char* dst = sm.ring + (size_t)g * kGroupBytes;
    mbar_expect_tx(&ctl.mbar[g], elems * 6);
    bulk_load(dst, rowp + e0 * 2, elems * 2, &ctl.mbar[g]);
    bulk_load(dst + kRwDenseElems * 2, nrowp + e0, elems * 4, &ctl.mbar[g]);
  };
  if (threadIdx.x == 0)
    for (int g = 0; g < kRwDenseGroups; ++g) issue(g, g);
  float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
  uint32_t b1 = 0;
  int t1 = 0x7FFFFFFF;
  int g = 0;
  ok = true;
  for (int c = 0; c < ngroups; ++c) {
    const bool arrived = mbar_wait_suspended(&ctl.mbar[g], (phases >> g) & 1u);
    phases ^= 1u << g;
    const unsigned char* buf = sm.ring + (size_t)g * kGroupBytes;
    const float* nbuf = reinterpret_cast<const float*>(buf + kRwDenseElems * 2);
    const int64_t rest = sp.vocab - (int64_t)c * kRwDenseElems;
    const int nvec = (int)((rest < kRwDenseElems ? rest : kRwDenseElems) >> 3);
#pragma unroll 1
    for (int v = threadIdx.x; v < nvec; v += kRwThreads) {
      const uint4 x = *reinterpret_cast<const uint4*>(buf + (size_t)v * 16);
      const __nv_bfloat162 m =
          __hmax2_nan(__hmax2_nan(bf162_bits(x.x), bf162_bits(x.y)), __hmax2_nan(bf162_bits(x.z), bf162_bits(x.w)));
      if (!__hblt2(m, tv2)) {
        // eight independent screened scores, then their best two
        const uint32_t wd[4] = {x.x, x.y, x.z, x.w};
        const float4 n0 = *reinterpret_cast<const float4*>(nbuf + v * 8);
        const float4 n1 = *reinterpret_cast<const float4*>(nbuf + v * 8 + 4);
        const float un[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
        float sc[8];
        float v1 = -INFINITY, v2 = -INFINITY;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t hi = (e & 1) ? (wd[e >> 1] & 0xFFFF0000u) : (wd[e >> 1] << 16);
          const float xf = __uint_as_float(hi);
          sc[e] = !(xf < tvf) ? fmaf(xf, inv_T, gumbel_screen(un[e])) : -INFINITY;
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
          t1 = c * kRwDenseElems + v * 8 + ebest;
        }
        a2 = fmaxf(fminf(a1, v1), fmaxf(a2, v2));
        a1 = fmaxf(a1, v1);
      }
    }
    if (__syncthreads_or(!arrived)) { ok = false; return 0; }
    if (threadIdx.x == 0) issue(c + kRwDenseGroups, g);
    if (++g == kRwDenseGroups) g = 0;
  }
  uint32_t bkey;
  int btok;
  rw_block_top(a1, t1, ctl, bkey, btok);
  const float amax = key_f32(bkey);
  const float cut = amax - (kGumbelSlack + 1e-5f * fabsf(amax));
  const bool have = t1 != 0x7FFFFFFF;
  const bool mine = have && f32_key(a1) == bkey && t1 == btok;
  const int multi = __syncthreads_or((have && !mine && a1 >= cut) || a2 >= cut);
  if (!multi) return btok == 0x7FFFFFFF ? 0 : btok;
  const int crowded = __syncthreads_or(a2 >= cut);
  Best best{-INFINITY, 0x7FFFFFFF};
  if (!crowded) {
    if (have && a1 >= cut) best = Best{__fdiv_rn(__uint_as_float(b1 << 16), T_) + gumbel_exact(u1), t1};
  } else {
    // a thread holds two contenders (there may be a third): look at the row again, from global memory
    const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(rowp);
    for (int64_t c = threadIdx.x; c < sp.vocab; c += kRwThreads) {
      const float x = __uint_as_float((uint32_t) * reinterpret_cast<const unsigned short*>(rp + c) << 16);
      if (!(x < tvf)) {
        const float u = sp.noise.at(nrow, c);
        if (fmaf(x, inv_T, gumbel_screen(u)) >= cut) best = best_of(best, Best{__fdiv_rn(x, T_) + gumbel_exact(u), (int)c});
      }
    }
  }
  rw_block_top(best.y, best.tok, ctl, bkey, btok);
  return btok == 0x7FFFFFFF ? 0 : btok;
}

// Dynamic shared memory: kRwSmemBytes.  Two CTAs per SM.
__global__ void __launch_bounds__(kRwThreads, 2) sample_rows_stream_kernel(RowsParams p) {
  extern __shared__ __align__(128) unsigned char rw_smem[];
  RwSmem sm;
  sm.ring = rw_smem;
  sm.hist = reinterpret_cast<uint32_t*>(rw_smem + kRwRingBytes);
  sm.tok = sm.hist + kRwBins;
  sm.bits = reinterpret_cast<unsigned short*>(sm.tok + kRwCap);
  sm.vlist = sm.bits + kRwCap;
  sm.ctl = reinterpret_cast<RwControl*>(reinterpret_cast<unsigned char*>(sm.vlist) + kRwListBytes);
  RwControl& ctl = *sm.ctl;
  // scratch of the whole-row routines, over the ring (idle whenever they run)
  SelectShared& s = *reinterpret_cast<SelectShared*>(rw_smem);
  uint64_t* cand = reinterpret_cast<uint64_t*>(rw_smem + kSharedHeader);
  uint32_t* win = reinterpret_cast<uint32_t*>(rw_smem + kSharedHeader);
  const SampleParams& sp = p.sp;
  const int lane = lane_id(), warp = warp_id();
  const int64_t V = sp.vocab;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRwSlots; ++i) mbar_init(&ctl.mbar[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  uint32_t phases = 0;
  uint32_t* wtok = sm.tok + warp * kRwWarpCap;
  unsigned short* wbits = sm.bits + warp * kRwWarpCap;
  unsigned short* wl = sm.vlist + warp * 32 * kRwVecPerThread;

  for (int64_t row = blockIdx.x; row < sp.rows; row += gridDim.x) {
    const unsigned char* rowp = reinterpret_cast<const unsigned char*>(sp.logits) + row * sp.row_stride * 2;
    const int64_t nrow = row + sp.dim0_offset;
    TLX_STAMP(sp, 0);
    // ---- the ring's first copies, then the parameters while they fly
    if (threadIdx.x == 0)
      for (int sl = 0; sl < kRwSlots; ++sl) rw_issue(p, rowp, sl, sm, sl);
    int K = sp.top_k[row];
    const float T_ = sp.temperature[row];
    const float pp = sp.top_p[row];
    if (K <= 0 || (int64_t)K >= V) K = (int)V;
    if (T_ < kSamplingEps) K = 1;   // greedy: the top candidate
    int cls;
    if (K <= kStMaxK) cls = kRwNormal;
    else if ((int64_t)K >= V) cls = pp < 1.0f ? kRwWide : kRwPlain;
    else cls = kRwOther;
    if (cls == kRwPlain && !p.dense_noise) cls = kRwOther;
    for (int i = threadIdx.x; i < kRwBins; i += kRwThreads) sm.hist[i] = 0;
    int key16 = 0;
    if (cls == kRwNormal || cls == kRwWide) {
      // the sample: 4096 elements out of the first two chunks requested (the visiting order spreads them
      // over the row); the later copies keep arriving while the threshold is worked out
      const int primed_chunks = p.nchunks < 2 ? p.nchunks : 2;
      uint32_t key[kRwKeys];
#pragma unroll
      for (int j = 0; j < kRwKeys / 8; ++j) {
        const int idx = (int)threadIdx.x + j * kRwThreads;   // 512 sample vectors
        const int sl = idx % primed_chunks;
        mbar_wait_suspended(&ctl.mbar[sl], (phases >> sl) & 1u);   // the pass waits for it again (and checks)
        const int nvec = rw_chunk_of(p, sl) == p.nchunks - 1 ? p.last_nvec : kRwChunkVecs;
        int v = (idx / primed_chunks) * (kRwChunkVecs * primed_chunks / 512);
        v = v < nvec ? v : v % nvec;
        const uint4 x = *reinterpret_cast<const uint4*>(sm.ring + (size_t)sl * kRwChunk + (size_t)v * 16);
        const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) key[j * 8 + e] = bf16_key16((e & 1) ? (w4[e >> 1] >> 16) : (w4[e >> 1] & 0xFFFFu));
      }
      int r = 1;   // wide rows: the sample's maximum
      if (cls == kRwNormal) {
        // rank in the sample that leaves, with four standard deviations of margin, at least K elements of
        // the row at or above the sample's element of that rank
        const float mu = (float)K * (float)kStSample / (float)V;
        r = (int)(mu + 4.0f * sqrtf(mu) + 2.999f);
        if ((float)r * (float)V / (float)kStSample > 0.8f * (float)kRwCap) cls = kRwOther;   // too many candidates
        r = r > kStSample ? kStSample : r;
      }
      key16 = rw_select_key(key, r, sm.tok, ctl);
      if (key16 > 0xFF80) cls = kRwOther;   // NaNs in the sample: the whole-row routines know what to do
      else if (cls == kRwWide) key16 = min(key16 + kStWinExtra, 0xFF80);
    }
    __syncthreads();   // histogram cleared, class and key settled
    TLX_STAMP(sp, 1);

    int status = cls == kRwNormal ? 0 : (int)kStatusGeneral;
    int tok = -1;
    bool ok = true;
    bool primed = true;   // the ring holds the row's first chunks
    if (cls == kRwNormal) {
      const uint32_t tbits = key16_bf16_bits((uint32_t)key16);
      const __nv_bfloat162 tv2 = bf162_splat_bits(tbits);
      const float tvf = __uint_as_float(tbits << 16);
      int wc = 0;
      ok = rw_pass(p, rowp, sm, phases, true, [&](const unsigned char* buf, int nvec, int c, bool full) {
        if (wc > kRwWarpCap) return;   // the list has overflowed: the tail will see it
        if (full) rw_filter_chunk<true>(buf, nvec, c * kRwChunkElems, tvf, tv2, wtok, wbits, wc, wl);
        else rw_filter_chunk<false>(buf, nvec, c * kRwChunkElems, tvf, tv2, wtok, wbits, wc, wl);
      });
      primed = false;
      TLX_STAMP(sp, 2);
      if (ok && sp.noise.dense && T_ >= kSamplingEps) {
        // most of the candidates' noise is wanted two microseconds from now: start it on its way to L2
        const float* nr = sp.noise.dense_row(nrow);
        const int n = wc < kRwWarpCap ? wc : kRwWarpCap;
        for (int i = lane; i < n; i += 32) prefetch_l2(nr + wtok[i]);
      }
      if (ok) tok = rw_tail_normal(sp, nrow, K, key16, pp, T_, sm, wc);
      TLX_STAMP(sp, 3);
#ifdef TLX_TIMELINE_TWICE
      __syncthreads();
      for (int i = threadIdx.x; i < kRwBins; i += kRwThreads) sm.hist[i] = 0;
      __syncthreads();
      if (ok) tok = rw_tail_normal(sp, nrow, K, key16, pp, T_, sm, wc);
      TLX_STAMP(sp, 5);
#endif
    } else if (cls == kRwWide) {
      const float xref = key16_value(key16);
      const float nxl = -xref * 1.44269504f;
      float lump = 0.f;
      int above = 0;
      uint32_t dmin = 0xFFFFFFFFu;   // (the greatest element's position is not used on this path)
      ok = rw_pass(p, rowp, sm, phases, true, [&](const unsigned char* buf, int nvec, int, bool full) {
        if (full) st_hist_chunk<true, kRwThreads, kRwVecPerThread>(buf, nvec, key16, nxl, sm.hist, lump, above, 0, dmin);
        else st_hist_chunk<false, kRwThreads, kRwVecPerThread>(buf, nvec, key16, nxl, sm.hist, lump, above, 0, dmin);
      });
      primed = false;
      TLX_STAMP(sp, 2);
      if (ok) {
        // the row's maximum, denominator and threshold key from the window and the sum below it
        const int bad = __syncthreads_or(above < 0 || !(lump >= 0.f));
        int vstar = -1;
        if (!bad) vstar = wide_threshold_core<kRwThreads>(key16, pp, sm.hist, (double)lump, 0, ctl.wide);
        TLX_STAMP(sp, 4);
        if (vstar >= 0) {
          // how many elements are kept (their keys are at or above the threshold key)
          uint32_t nk = 0;
          for (int i = threadIdx.x; i <= key16 - vstar && i < kRwBins; i += kRwThreads) nk += sm.hist[i];
          nk = __reduce_add_sync(0xFFFFFFFFu, nk);
          __syncthreads();
          if (lane == 0) ctl.red[warp] = (int)nk;
          __syncthreads();
          int nkept = 0;
          for (int w = 0; w < kRwWarps; ++w) nkept += ctl.red[w];
          const uint32_t tbits = key16_bf16_bits((uint32_t)vstar);
          const __nv_bfloat162 tv2 = bf162_splat_bits(tbits);
          const float tvf = __uint_as_float(tbits << 16);
          if (nkept <= kRwCap / 2 || !p.dense_noise) {
            // second pass with the candidate filter at the threshold: the lists hold exactly the kept elements
            int wc = 0;
            ok = rw_pass(p, rowp, sm, phases, false, [&](const unsigned char* buf, int nvec, int c, bool full) {
              if (wc > kRwWarpCap) return;
              if (full) rw_filter_chunk<true>(buf, nvec, c * kRwChunkElems, tvf, tv2, wtok, wbits, wc, wl);
              else rw_filter_chunk<false>(buf, nvec, c * kRwChunkElems, tvf, tv2, wtok, wbits, wc, wl);
            });
            const int over = __syncthreads_or(wc > kRwWarpCap);
            TLX_STAMP(sp, 5);
            if (ok && !over) {
              RwKeep keep{};
              keep.all = true;
              tok = rw_score_lists(sp, nrow, T_, keep, sm, wc);
            }
          } else {
            tok = rw_dense_pass(p, row, T_, tvf, tv2, sm, phases, ok);
          }
        }
      }
    } else if (cls == kRwPlain) {
      // the copies requested at the start are not used (the dense pass arranges the ring differently)
      ok = rw_drain(p, sm, phases);
      primed = false;
      const __nv_bfloat162 all2 = bf162_splat_bits(0x7FC0u);
      if (ok) tok = rw_dense_pass(p, row, T_, __uint_as_float(0x7FC00000u), all2, sm, phases, ok);
    }
    if (ok && tok < 0) {
      // whole-row routines (exact, slow): the ring must be idle, it becomes their scratch
      if (primed) ok = rw_drain(p, sm, phases);
      __syncthreads();
      if (ok) {
        const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(rowp);
        if (cls == kRwNormal) {
          status |= kStatusRedone;
          exact_select_row<TLX_BF16>(rp, V, K, s, cand);
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
                  K, pp, T_, s, [&](int i) { return key_f32(cand_key(cand[i])); },
                  [&](int i) { return (int)cand_low(cand[i]); },
                  [&](int i) { return sp.noise.at(nrow, (int64_t)cand_low(cand[i])); });
            }
          }
        } else if ((int64_t)K >= V && pp >= 1.0f) {
          tok = final_argmax<TLX_BF16>(rp, V, T_, 0u, false, 0u, 0u, false, sp.noise, nrow, s);
        } else {
          if (cls == kRwWide) status |= kStatusRedone;
          RowPreset none;
          tok = general_row_bf16<kWin>(rp, V, K, pp, T_, sp.noise, nrow, s, win, none);
        }
      }
      __syncthreads();
    }
    TLX_STAMP(sp, 8);
    if (threadIdx.x == 0 && sp.timeline) sp.timeline[(size_t)blockIdx.x * 16 + 9] = cls;
    if (threadIdx.x == 0) {
      if (!ok) status |= kStatusTimeout;
      sp.out_tokens[row] = ok ? tok : 0;
      if (sp.out_status) sp.out_status[row] = status;
    }
    if (!ok) return;   // a copy never arrived: the barriers' phases are unknown now
    __syncthreads();
  }
}

}  // namespace tlx
