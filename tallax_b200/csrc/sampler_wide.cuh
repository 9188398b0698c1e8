// Rows without a top-k filter ("wide" rows), bf16: one thread-block cluster per row keeps the
// whole row resident in the shared memory of its CTAs, so the row is read from HBM once although
// it is looked at three times (maximum, histogram, final arg-max).
//
//   1. every CTA brings its contiguous share of the row in with bulk copies, takes the share's
//      maximum; the cluster agrees on the row maximum through distributed shared memory;
//   2. every CTA histograms its share over the window of 16-bit keys below the row maximum and
//      sums exp(x - max) of what lies below the window;
//   3. the CTAs add the histograms up (each one an eighth of the bins) and look, each in its
//      eighth, for the bin at which the cumulative mass count * exp(value - max) reaches
//      top_p times the denominator: the top-p threshold;
//   4. every CTA takes the Gumbel arg-max over the kept elements of its share (noise read with
//      coalesced 16-byte loads), decides its winner on the f64-evaluated Gumbel term, and rank 0
//      picks the best of the winners.
// Included by sampler.cu after the helpers it uses.
#pragma once
#include <cooperative_groups.h>

namespace tlx {

constexpr int kWideCluster = 8;
constexpr int kWidePartBytes = 65536;               // largest share of a row one CTA holds
constexpr int kWideBinsPer = kWin / kWideCluster;   // bins each CTA adds up over the cluster
static_assert(kWideBinsPer == kThreads, "one combined bin per thread");

struct __align__(16) WideExchange {   // what the CTAs of a cluster read from one another
  uint32_t kmax32;
  int timeout;
  double below;                       // sum of exp(x - row max) over this CTA's elements below the window
  double mass;                        // mass of this CTA's share of the combined bins
  unsigned long long best;            // f32 key of the exact score << 32 | (0x7FFFFFFF - token)
  float top_a;                        // best screened score of this CTA's share and its token
  int top_tok;
  int leaders;                        // contenders in this CTA's share (2 = more than can be told apart)
  uint32_t found;                     // key + 1 of the threshold bin if it lies in this CTA's share of the bins
};

struct __align__(16) WideControl {
  unsigned long long mbar;
  int timeout;
  int list[kThreads];
};

constexpr size_t kWideSmem = kSharedHeader + (size_t)kWin * 4 + sizeof(WideExchange) + sizeof(WideControl) + 128 +
                             (size_t)kWidePartBytes;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __cluster_dims__(kWideCluster, 1, 1) __launch_bounds__(kThreads, 2)
    sample_wide_rows_kernel(SampleParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  uint32_t* win = reinterpret_cast<uint32_t*>(smem_raw + kSharedHeader);
  WideExchange& xch = *reinterpret_cast<WideExchange*>(smem_raw + kSharedHeader + (size_t)kWin * 4);
  WideControl& ctl = *reinterpret_cast<WideControl*>(smem_raw + kSharedHeader + (size_t)kWin * 4 + sizeof(WideExchange));
  unsigned char* part = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(&ctl) + sizeof(WideControl) + 127) & ~uintptr_t(127));

  const int rank = (int)cluster.block_rank();
  const int ncl = (int)gridDim.x / kWideCluster, cid = (int)blockIdx.x / kWideCluster;
  const int64_t n = p.vocab;
  const int nvec_row = (int)(n >> 3);                       // the row is a whole number of 16-byte vectors
  const int vper = (nvec_row + kWideCluster - 1) / kWideCluster;
  const int v0 = rank * vper;
  const int myvec = max(0, min(vper, nvec_row - v0));
  const uint4* vp = reinterpret_cast<const uint4*>(part);
  const bool noise_vec = p.noise.dense && ((reinterpret_cast<uintptr_t>(p.noise.dense) & 15) == 0) &&
                         ((p.noise.stride & 3) == 0);

  if (threadIdx.x == 0) {
    mbar_init(&ctl.mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl.timeout = 0;
  }
  __syncthreads();
  uint32_t phase = 0;
  int seen = 0;   // wide rows before the current block of rows

  for (int64_t base = 0; base < p.rows; base += kThreads) {
    // The wide rows are dealt to the clusters round-robin; every CTA of a cluster derives the
    // same list (positions are computed, not claimed, so the order is the same everywhere).
    const int64_t r = base + threadIdx.x;
    bool wide = false;
    if (r < p.rows) {
      int K;
      // rows with top_p >= 1 need no histogram: the rows kernel streams them
      wide = classify_row(p, r, K) == (int)kGeneral && (int64_t)K >= n && p.top_p[r] < 1.0f;
    }
    uint32_t total;
    const uint32_t incl = block_scan_incl<uint32_t>(wide ? 1u : 0u, s.scan_u32, &total, ShflUpU32());
    const int first = seen + ((cid - seen % ncl) + ncl) % ncl;   // first wide index of this cluster in the block
    const int end = seen + (int)total;
    const int ln = end > first ? (end - 1 - first) / ncl + 1 : 0;
    if (wide) {
      const int idx = seen + (int)incl - 1;
      if (idx >= first && (idx - first) % ncl == 0) ctl.list[(idx - first) / ncl] = (int)threadIdx.x;
    }
    seen = end;
    __syncthreads();

    for (int j = 0; j < ln; ++j) {
      const int64_t row = base + ctl.list[j];
      const int64_t nrow = row + p.dim0_offset;
      const float pp = p.top_p[row], T_ = p.temperature[row];
      const __nv_bfloat16* rowp = reinterpret_cast<const __nv_bfloat16*>(p.logits) + row * p.row_stride;

      // ---- 1. the share comes in; row maximum -------------------------------------------
      if (warp_id() == 0 && myvec > 0) {
        const uint32_t bytes = (uint32_t)myvec * 16u;
        if (lane_id() == 0) mbar_expect_tx(&ctl.mbar, bytes);
        __syncwarp();
        const unsigned char* src = reinterpret_cast<const unsigned char*>(rowp) + (size_t)v0 * 16;
        for (uint32_t off = (uint32_t)lane_id() * 4096u; off < bytes; off += 32u * 4096u)
          bulk_load(part + off, src + off, min(4096u, bytes - off), &ctl.mbar);
      }
      if (myvec > 0) {
        if (!mbar_wait(&ctl.mbar, phase)) ctl.timeout = 1;
        phase ^= 1u;
      }
      const uint32_t tkey = thread_max_key<TLX_BF16>(part, myvec, 1 << 30);
      const uint32_t my_kmax32 = block_max_u32(tkey, s.scan_u32);
      if (threadIdx.x == 0) xch.kmax32 = my_kmax32;
      cluster.sync();
      uint32_t kmax32 = 0;
#pragma unroll
      for (int c = 0; c < kWideCluster; ++c) {
        const uint32_t k = cluster.map_shared_rank(&xch, c)->kmax32;
        kmax32 = k > kmax32 ? k : kmax32;
      }
      const int kmax = (int)(kmax32 >> 16);
      const float xmax = key_f32(kmax32);

      // ---- 2./3. threshold (top_p >= 1 keeps the whole row) -------------------------------
      // The threshold is looked for window by window: first the kWin keys below the row maximum,
      // then, if the cumulative mass has not reached top_p * Z there, the kWin keys below the
      // largest key that is present under that window, and so on.  Every further window costs two
      // more passes over the resident share, none over global memory.
      int vstar16 = 0;
      if (pp < 1.0f) {
        const float neg_xmax_l2e = -xmax * 1.44269504f;
        int whi = kmax;
        double cum = 0.0, target = 0.0;
        for (int round = 0;; ++round) {
          for (int i = threadIdx.x; i < kWin; i += blockDim.x) win[i] = 0;
          __syncthreads();
          float below = 0.f;
          if (round == 0 && kmax >= 0x8000 + kWin) {
            // positive maximum (the usual case): every negative element is below the window, and one
            // unsigned compare of (kmax - 0x8000) - h against the window size decides for the others
            const uint32_t dpos = (uint32_t)(kmax - 0x8000);
            auto visit = [&](uint32_t h, float x) {
              const uint32_t d = dpos - h;
              if (d < (uint32_t)kWin) atomicAdd(&win[d], 1u);
              else below += ex2_approx(fmaf(x, 1.44269504f, neg_xmax_l2e));
            };
            for (int i = threadIdx.x; i < myvec; i += blockDim.x) {
              const uint4 v = vp[i];
              const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                visit(w4[q] & 0xFFFFu, __uint_as_float(w4[q] << 16));
                visit(w4[q] >> 16, __uint_as_float(w4[q] & 0xFFFF0000u));
              }
            }
          } else {
            auto visit = [&](uint32_t h) {
              const uint32_t k16 = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);
              const int d = whi - (int)k16;
              if (d < kWin) { if (d >= 0) atomicAdd(&win[d], 1u); }
              else if (round == 0) below += ex2_approx(fmaf(__uint_as_float(h << 16), 1.44269504f, neg_xmax_l2e));
            };
            for (int i = threadIdx.x; i < myvec; i += blockDim.x) {
              const uint4 v = vp[i];
              const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) { visit(w4[q] & 0xFFFFu); visit(w4[q] >> 16); }
            }
          }
          if (round == 0) {
            double below_cta;
            block_scan_incl<double>((double)below, s.scan_f64, &below_cta, ShflUpF64());
            if (threadIdx.x == 0) xch.below = below_cta;
          }
          cluster.sync();
          // This CTA's eighth of the bins, summed over the cluster, and the running mass inside it.
          // The search for the bin at which the cumulative mass reaches the target is distributed
          // the same way: bin t of CTA r covers the interval (B_r + incl[t-1], B_r + incl[t]], with
          // B_0 = cum and B_{r+1} = B_r + mass_r evaluated in this order by everybody, so that the
          // intervals tile the line exactly and at most one bin claims the target.
          double* incl_of = reinterpret_cast<double*>(win);   // once everybody has read it, this CTA's histogram may go
          {
            const int bin = rank * kWideBinsPer + (int)threadIdx.x;
            uint32_t c = 0;
#pragma unroll
            for (int q = 0; q < kWideCluster; ++q) c += cluster.map_shared_rank(win, q)[bin];
            const double m = (c && whi - bin >= 0) ? (double)c * (double)expf(key16_value(whi - bin) - xmax) : 0.0;
            double mass_cta;
            const double incl = block_scan_incl<double>(m, s.scan_f64, &mass_cta, ShflUpF64());
            if (threadIdx.x == 0) { xch.mass = mass_cta; xch.found = 0; }
            cluster.sync();   // everybody has read everybody's histogram, the masses are out
            incl_of[threadIdx.x] = incl;
            double b_r = cum, b_all = cum, zb = 0.0;
#pragma unroll
            for (int q = 0; q < kWideCluster; ++q) {
              const WideExchange* o = cluster.map_shared_rank(&xch, q);
              if (q == rank) b_r = b_all;
              b_all += o->mass;
              zb += o->below;
            }
            if (round == 0) target = (double)pp * ((b_all - cum) + zb);
            __syncthreads();
            const double lo_m = b_r + (threadIdx.x ? incl_of[threadIdx.x - 1] : 0.0);
            const double hi_m = b_r + incl;
            if (m > 0.0 && lo_m < target && hi_m >= target) xch.found = (uint32_t)(whi - bin) + 1u;
            cum = b_all;
          }
          cluster.sync();
          uint32_t found1 = 0;   // key + 1
#pragma unroll
          for (int q = 0; q < kWideCluster; ++q) {
            const uint32_t f = cluster.map_shared_rank(&xch, q)->found;
            found1 = f > found1 ? f : found1;
          }
          const int found = (int)found1 - 1;
          if (found >= 0) { vstar16 = found; break; }
          // the next window hangs from the largest key that is present below this one
          const int lo = whi - kWin;
          if (lo < 0) break;
          uint32_t next = 0;   // key + 1, 0 = nothing below
          for (int i = threadIdx.x; i < myvec; i += blockDim.x) {
            const uint4 v = vp[i];
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const uint32_t h = (q & 1) ? (w4[q >> 1] >> 16) : (w4[q >> 1] & 0xFFFFu);
              const uint32_t k16 = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);
              if ((int)k16 <= lo && k16 + 1 > next) next = k16 + 1;
            }
          }
          next = block_max_u32(next, s.scan_u32);
          if (threadIdx.x == 0) xch.kmax32 = next;
          cluster.sync();
          next = 0;
#pragma unroll
          for (int q = 0; q < kWideCluster; ++q) {
            const uint32_t k = cluster.map_shared_rank(&xch, q)->kmax32;
            next = k > next ? k : next;
          }
          if (next == 0) break;   // nothing left: the whole row is kept
          whi = (int)next - 1;
        }
      }

      // ---- 4. Gumbel arg-max over the kept elements of the share ---------------------------
      const uint32_t min_key = vstar16 == 0 ? 0u : key16_to_key32((uint32_t)vstar16);
      const float thr = vstar16 == 0 ? -INFINITY : key16_value(vstar16);
      const __nv_bfloat162 thr2 = __float2bfloat162_rn(thr);
      const float inv_T = 1.0f / T_;
      float a1 = -INFINITY, a2 = -INFINITY, u1 = 0.5f;
      uint32_t k1 = 0;
      int c1 = 0x7FFFFFFF;
      // Vectors with a kept element are rare for a small nucleus and the rule for a large one, so the
      // noise of a batch of vectors is requested before any of it is used: one memory latency per
      // batch instead of one per vector.
      constexpr int kBatch = 2;
      auto pass_over = [&](float cut, Best* exact) {
        for (int i0 = threadIdx.x; i0 < myvec; i0 += kBatch * (int)blockDim.x) {
          uint4 v[kBatch];
          float4 nz[kBatch][2];
          bool some[kBatch];
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            const int i = i0 + b * (int)blockDim.x;
            some[b] = false;
            if (i < myvec) {
              v[b] = vp[i];
              const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(v[b].x), bf162_bits(v[b].y)),
                                                   __hmax2_nan(bf162_bits(v[b].z), bf162_bits(v[b].w)));
              some[b] = !__hblt2(m, thr2);   // something kept in this vector
            }
            if (some[b] && noise_vec) {
              const float4* np4 =
                  reinterpret_cast<const float4*>(p.noise.dense_row(nrow) + ((int64_t)(v0 + i) << 3));
              nz[b][0] = __ldg(np4);
              nz[b][1] = __ldg(np4 + 1);
            }
          }
#pragma unroll
          for (int b = 0; b < kBatch; ++b) {
            if (some[b]) {
              const int64_t col0 = (int64_t)(v0 + i0 + b * (int)blockDim.x) << 3;
              auto consider = [&](uint32_t bits, float un, int q) {
                const float x = __uint_as_float(bits);
                const uint32_t key = f32_key(x);
                if (key >= min_key) {
                  const float u = noise_vec ? un : p.noise.at(nrow, col0 + q);
                  const float a = x * inv_T + gumbel_screen(u);
                  if (exact) {
                    if (a >= cut) *exact = best_of(*exact, Best{__fdiv_rn(x, T_) + gumbel_exact(u), (int)(col0 + q)});
                  } else if (a > a1) { a2 = a1; a1 = a; k1 = key; u1 = u; c1 = (int)(col0 + q); }
                  else if (a > a2) a2 = a;
                }
              };
              consider(v[b].x << 16, nz[b][0].x, 0);
              consider(v[b].x & 0xFFFF0000u, nz[b][0].y, 1);
              consider(v[b].y << 16, nz[b][0].z, 2);
              consider(v[b].y & 0xFFFF0000u, nz[b][0].w, 3);
              consider(v[b].z << 16, nz[b][1].x, 4);
              consider(v[b].z & 0xFFFF0000u, nz[b][1].y, 5);
              consider(v[b].w << 16, nz[b][1].z, 6);
              consider(v[b].w & 0xFFFF0000u, nz[b][1].w, 7);
            }
          }
        }
      };
      // The noise of the kept vectors is at scattered places of a tensor far larger than the L2: ask
      // for all of it first, so that the pass below waits for the L2 and not for HBM, vector by vector.
      if (noise_vec) {
        for (int i = threadIdx.x; i < myvec; i += blockDim.x) {
          const uint4 v = vp[i];
          const __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(bf162_bits(v.x), bf162_bits(v.y)),
                                               __hmax2_nan(bf162_bits(v.z), bf162_bits(v.w)));
          if (!__hblt2(m, thr2))
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.noise.dense_row(nrow) + ((int64_t)(v0 + i) << 3)));
        }
      }
      pass_over(0.f, nullptr);
      // The CTAs agree on the best screened score of the row; what lies within the slack below it
      // are the contenders.  A single contender wins as it stands; otherwise each CTA decides its
      // contenders on the f64-evaluated Gumbel term and rank 0 takes the best of those.
      const Best top_cta = block_best(Best{a1, c1}, s);
      if (threadIdx.x == 0) {
        xch.top_a = top_cta.y;
        xch.top_tok = top_cta.tok;
      }
      cluster.sync();
      Best top{-INFINITY, 0x7FFFFFFF};
#pragma unroll
      for (int q = 0; q < kWideCluster; ++q) {
        const WideExchange* o = cluster.map_shared_rank(&xch, q);
        top = best_of(top, Best{o->top_a, o->top_tok});
      }
      const float cut = top.y - (kGumbelSlack + 1e-5f * fabsf(top.y));
      const int leaders = __syncthreads_count(a1 >= cut);
      const int crowded = __syncthreads_or(a2 >= cut);
      Best best{-INFINITY, 0x7FFFFFFF};
      if (crowded) {
        pass_over(cut, &best);   // a thread saw two contenders: look again and decide exactly
      } else if (a1 >= cut) {
        best = Best{__fdiv_rn(key_f32(k1), T_) + gumbel_exact(u1), c1};
      }
      if (leaders > 0 || crowded) best = block_best(best, s);
      if (threadIdx.x == 0) {
        xch.best = best.tok != 0x7FFFFFFF
                       ? (((unsigned long long)f32_key(best.y) << 32) | (uint32_t)(0x7FFFFFFF - best.tok))
                       : 0ull;
        xch.leaders = crowded ? 2 : leaders;
        xch.timeout = ctl.timeout;
      }
      cluster.sync();
      if (rank == 0 && threadIdx.x == 0) {
        unsigned long long b = 0;
        int timeout = 0, contenders = 0;
        for (int q = 0; q < kWideCluster; ++q) {
          const WideExchange* o = cluster.map_shared_rank(&xch, q);
          b = o->best > b ? o->best : b;
          timeout |= o->timeout;
          contenders += o->leaders;
        }
        p.out_tokens[row] = contenders == 1 ? top.tok : 0x7FFFFFFF - (int32_t)(uint32_t)b;
        if (p.out_status) p.out_status[row] = kStatusGeneral | (timeout ? kStatusTimeout : 0);
      }
      // The next row's exchanges are fenced by its own cluster barriers: a CTA rewrites a field
      // only after a barrier that every reader of the old value has passed.
    }
    __syncthreads();
  }
  cluster.sync();   // no CTA exits while another may still read its shared memory
}

}  // namespace tlx
