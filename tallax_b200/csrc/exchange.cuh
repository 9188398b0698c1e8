// Candidate exchange of the vocab-sharded sampler over peer memory (NVLink / NVSwitch).
//
// Every rank owns one exchange buffer of the same layout and maps the buffers of the other ranks.  The
// candidate kernel of rank s stores each row's block straight into slot s of EVERY rank's buffer (plain
// peer stores) and then adds one to that row's arrival word there (a system-scope release).  The merge
// kernel on a rank waits, per row and with a bounded spin, until the row's arrival word reads `world`,
// merges the row out of its own memory and clears the word.  No collective call and no host round trip
// lies between the two kernels.
//
// Two sets of (arrival words, candidate slots) alternate from step to step: a rank can run at most one
// step ahead of any other (its next merge needs every rank's next candidates), so what it writes for
// step t + 1 never meets what a slower rank still reads for step t.  The set of a step is the low bit of
// a step counter in the buffer's header, advanced by the merge kernel's last CTA: CUDA-graph replays and
// eager calls need no host-side bookkeeping.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace tlx {

constexpr int kExchangeMaxWorld = 16;

struct ExchangeHeader {
  uint32_t step;     // steps completed on this rank; its low bit selects the set
  uint32_t done;     // merge CTAs that finished in the current step
  uint32_t error;    // 1 once a wait gave up, 2 once a call's extents did not match the buffer's
  uint32_t rows, k_cand, world;   // what the buffer was made for (tlx_exchange_create); the kernels check it
  uint32_t pad[58];
};
static_assert(sizeof(ExchangeHeader) == 256, "header is one 256-byte block");

struct ExchangeLayout {
  size_t off_flags[2];   // uint32_t [rows]
  size_t off_cand[2];    // float [world][3][rows][k]: values, token ids (int32 bits), noise
  size_t block_elems;    // 3 * rows * k
  size_t bytes;
};

inline __host__ __device__ ExchangeLayout exchange_layout(int64_t rows, int k, int world) {
  ExchangeLayout l{};
  size_t o = sizeof(ExchangeHeader);
  l.block_elems = (size_t)3 * (size_t)rows * (size_t)k;
  for (int q = 0; q < 2; ++q) {
    l.off_flags[q] = o;
    o += ((size_t)rows * 4 + 255) & ~(size_t)255;
    l.off_cand[q] = o;
    o += ((size_t)world * l.block_elems * 4 + 255) & ~(size_t)255;
  }
  l.bytes = o;
  return l;
}

// What the candidate kernel needs to deliver a row to every rank.
struct ExchangeTargets {
  unsigned char* peer[kExchangeMaxWorld];   // the ranks' buffers as mapped here; [rank] is this rank's own
  int world;                                // 0: no exchange, results go to the caller's arrays
  int rank;
  size_t off_flags[2], off_cand[2];
};

}  // namespace tlx
