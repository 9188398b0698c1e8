/* tallax_b200 -- C ABI of the B200 (sm_100a) row-wise select / sort / sample library.
 *
 * Every entry point
 *   - takes raw device pointers, sizes and a CUDA stream (passed as void* so that
 *     this header needs no CUDA include);
 *   - only enqueues work on that stream: no allocation, no synchronisation, no host
 *     read of device data (scratch memory is an explicit `workspace` argument whose
 *     size the matching `*_workspace_bytes` function reports);
 *   - returns TLX_OK or a negative error code; `tlx_last_error()` gives the message
 *     of the calling thread's last failure.  Device code never traps: waits are
 *     bounded and failures are reported through status words.
 *
 * The reference project (oliverdutton/tallax) has no C or FFI boundary: its device
 * boundary is the `pl.pallas_call` site of each operator.  Each declaration below
 * names the call site (path inside the reference project) that it replaces.
 */
#ifndef TALLAX_B200_H_
#define TALLAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TLX_ABI_VERSION 1

typedef enum {
  TLX_OK = 0,
  TLX_ERR_INVALID = -1,     /* bad argument (maps to ValueError)            */
  TLX_ERR_UNSUPPORTED = -2, /* valid but not built (NotImplementedError)    */
  TLX_ERR_WORKSPACE = -3,   /* workspace missing or too small               */
  TLX_ERR_CUDA = -4         /* a CUDA runtime call failed                   */
} tlx_status;

typedef enum {
  TLX_F32 = 0,
  TLX_BF16 = 1,
  TLX_I32 = 2,
  TLX_F16 = 3,
  TLX_U32 = 4
} tlx_dtype;

int tlx_abi_version(void);
const char* tlx_last_error(void);
/* Number of kernels this library has launched in the process so far (diagnostic: lets a
 * benchmark count launches per call instead of assuming them). */
unsigned long long tlx_kernel_launches(void);

/* Optional.  Touches `device` once (so that no later call makes its first query of the device
 * inside a stream capture) and, with TLX_INIT_SIDE_STREAM, creates the calling thread's helper
 * stream and events on it and lets tlx_sample use them.  Without this call the library creates no
 * CUDA stream or event of its own, ever.                                                       */
#define TLX_INIT_SIDE_STREAM 1u
int tlx_init(int device, unsigned flags);

/* Checked builds only (python -m tallax_b200.build --checked -> libtallax_b200_checked.so): the streaming
 * sampler's kernels verify the shared-memory and workspace indices they rely on, skip an access whose index
 * is out of range and record the first such event.  Synchronises the device, copies {violations, site,
 * index, bound} to out4 (nullable), clears the record, and returns 1 if there was a violation, 0 if not;
 * TLX_ERR_UNSUPPORTED in other builds.                                                               */
int tlx_debug_check_status(int32_t* out4);

/* ---- device operands -------------------------------------------------------------------------
 * A caller under a tracing compiler (an XLA custom call, a CUDA graph whose key changes between
 * replays) has the PRNG key and the batch offset only as device buffers.  The *_dev entry points
 * take them that way: key_dev points to the key's two uint32 words in device memory,
 * dim0_offset_dev (nullable = 0) to an int32 scalar in device memory; both are read by the kernels
 * when they run, never by the host.  Everything else is as in the entry point of the same name.
 * They replace the traced operands `rng_key` and `dim0_offset` of tallax/_src/sampling.py:185-208,
 * 246-252 and tallax/_src/sparse_random.py:43-94.                                               */

/* ---- gather --------------------------------------------------------------------
 * out[b,j] = values[b, idx[b,j]] (axis 1) or out[i,b] = values[idx[i,b], b] (axis 0);
 * an index outside [0, extent) yields 0, as the reference does.
 * Replaces tallax/_src/gather.py:76-83 (pallas_call of take_along_axis_refs).       */
int tlx_take_along_axis(void* stream, const void* values, const int32_t* indices, void* out,
                        int64_t val_rows, int64_t val_cols, int64_t idx_rows, int64_t idx_cols,
                        int elem_bytes, int axis);

/* ---- cumsum --------------------------------------------------------------------
 * Inclusive prefix sum along `axis` (0 or 1), optionally reversed.  dtype: F32, I32.
 * Replaces tallax/_src/cumsum.py:93-101.                                             */
int tlx_cumsum(void* stream, const void* in, void* out, int64_t rows, int64_t cols, int dtype,
               int axis, int reverse);

/* ---- arg-max with lowest-index tie break ---------------------------------------
 * out_idx[r] = arg-max over columns (axis 1) or out_idx[c] = arg-max over rows
 * (axis 0) in the order-preserving key domain.  The payload-carrying form of the
 * reference (tallax/_src/bitonic_top_k.py:43-97 max_arrays) is this index plus a
 * gather of every operand.                                                          */
int tlx_argmax(void* stream, const void* keys, int dtype, int64_t rows, int64_t cols, int axis,
               int32_t* out_idx);

/* ---- sort ----------------------------------------------------------------------
 * Stable row-wise argsort of one key array [rows, n] (dtype F32, BF16, F16, I32, U32),
 * ascending or descending; ties always keep ascending position.  If `in_perm` is
 * given, row r sorts key[r, in_perm[r, :]] and the result permutation is composed
 * with it (least-significant-key-first chaining gives multi-key sorts).
 * out_keys (nullable): the sorted keys, canonicalised (-0 -> +0, one NaN).
 * out_perm (nullable): int32 source column of every output position.
 * Replaces tallax/_src/sort.py:559-571 and :740-758 (the VMEM sort and the HBM
 * substage kernels behind `sort`, sort.py:768-929).                                 */
size_t tlx_sort_workspace_bytes(int64_t rows, int64_t n);
int tlx_sort(void* stream, const void* keys, int dtype, int64_t rows, int64_t n, int descending,
             const int32_t* in_perm, void* out_keys, int32_t* out_perm, void* workspace,
             size_t workspace_bytes);

/* ---- sort without any allocation ------------------------------------------------
 * Same operation and results as tlx_sort, for callers that have nowhere to get scratch
 * memory from: plugin hosts whose memory pool is owned by another runtime, or processes that
 * were handed a fixed memory budget and must not call cudaMalloc (nor have the library call it
 * for them).  The
 * scratch of the multi-tile path is a fixed area inside the library image (16 MiB, reported by
 * tlx_sort_static_max_bytes; every GPU that loads the library holds it until exit).
 *   - rows whose composites need more than that are rejected with TLX_ERR_INVALID and a
 *     message; nothing is launched;
 *   - the first call on a device looks up the area's device address (with that device
 *     current), a host-side query; later calls only launch kernels;
 *   - all calls share the one area and it keeps the previous call's contents; the kernels
 *     write every entry before reading it, so nothing needs clearing, but two calls that
 *     overlap on the GPU (different streams) race: serialise them;
 *   - no cudaMalloc, cudaFree or allocating library routine is called.
 * No counterpart in the reference (its XLA runtime owns all device memory).           */
size_t tlx_sort_static_max_bytes(void);
int tlx_sort_static(void* stream, const void* keys, int dtype, int64_t rows, int64_t n, int descending,
                    const int32_t* in_perm, void* out_keys, int32_t* out_perm);

/* ---- top-k ---------------------------------------------------------------------
 * Row-wise descending top-`k_max` of x[rows, n] (row stride in elements), ties broken
 * by lower index; out_vals keeps the input dtype, out_idx is int32, both [rows, k_max].
 * k_per_row (nullable, device int32[rows]) with use_replace != 0: positions >= k[row]
 * receive replace_val in out_vals.
 * mode 0 = exact.  mode 1 = single-pass only (the reference's guarantee_convergence=False
 * contract): rows whose candidate buffer overflowed are answered from the candidates
 * seen, out_valid[0] is cleared, out_depths[row] is the number of threshold
 * refinements and out_cutoff[row] (f32 for float input, i32 for int) the final
 * candidate threshold.  out_valid/out_depths/out_cutoff may be NULL in mode 0.
 * workspace (optional): with tlx_top_k_workspace_bytes(rows, n, k_max) bytes of scratch (non-zero
 * only for up to 16 rows of at least 16 384 elements) an exact call that asks for no diagnostics
 * cuts every row into parts, one CTA each, and merges the parts' candidates; without it one CTA
 * takes a whole row.  The results are the same.
 * Replaces tallax/_src/top_k.py:482-506 (top_dynamic_k) and
 * tallax/_src/bitonic_top_k.py:390-401 (bitonic_top_k).                             */
#define TLX_TOPK_MAX_K 2048
size_t tlx_top_k_workspace_bytes(int64_t rows, int64_t n, int k_max);
int tlx_top_k(void* stream, const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
              int k_max, const int32_t* k_per_row, int use_replace, double replace_val, int mode,
              void* out_vals, int32_t* out_idx, int32_t* out_valid, int32_t* out_depths,
              void* out_cutoff, void* workspace, size_t workspace_bytes);

/* ---- canonical keys ---------------------------------------------------------------
 * In place: every float of x[count] becomes what it is after the round trip through the
 * order-preserving key (-0 -> +0, every NaN -> the canonical NaN); integers are left alone.
 * The sort's first key leaves tlx_sort in this form; this is for the further keys of a
 * multi-key sort, which are gathered through the final permutation (tallax/_src/sort.py:834-839). */
int tlx_canonicalize_keys(void* stream, void* x, int dtype, int64_t count);

/* ---- counter-based noise -------------------------------------------------------
 * out[i] = max(minval, f * (maxval - minval) + minval), f the [0,1) float made from
 * x0^x1 of threefry2x32(key, (0, idx0[i]*dim1_size + idx1[i])).
 * Replaces tallax/_src/sparse_random.py:43-64.                                      */
int tlx_sparse_random_uniform(void* stream, uint32_t key0, uint32_t key1, const int32_t* idx0,
                              const int32_t* idx1, int64_t count, int64_t dim1_size, float minval,
                              float maxval, float* out);
/* The same with the key as a device operand (see "device operands" below). */
int tlx_sparse_random_uniform_dev(void* stream, const uint32_t* key_dev, const int32_t* idx0,
                                  const int32_t* idx1, int64_t count, int64_t dim1_size, float minval,
                                  float maxval, float* out);

/* ---- top-p mask ------------------------------------------------------------------
 * topk_logits, out: f32 [k, batch], column b sorted descending along axis 0; p: f32[batch].
 * Keeps entries >= the logit at index #(cumulative softmax mass < p) (0.0 if that index
 * is k, as the reference's out-of-range gather gives), others become replace_val.
 * Replaces tallax/_src/sampling.py:25-62 (top_p_mask inside the fused kernel).      */
int tlx_top_p_mask(void* stream, const float* topk_logits, const float* p, int k, int64_t batch,
                   double replace_val, float* out);

/* ---- Gumbel arg-max with indexed noise -----------------------------------------
 * logits f32 [rows, cols]; noise at element e is the threefry uniform (clamped to
 * [tiny, 1)) with counter idx0[e] * dim1_size + idx1[e].  out_pos[line] = position along
 * `axis` of max(logits - log(-log(u))), lower position on ties; one line per row
 * (axis 1) or per column (axis 0).
 * Replaces tallax/_src/sparse_random.py:68-94 (sparse_random_categorical).          */
int tlx_gumbel_argmax(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1,
                      int64_t rows, int64_t cols, uint32_t key0, uint32_t key1, int64_t dim1_size,
                      int axis, int32_t* out_pos);
int tlx_gumbel_argmax_dev(void* stream, const float* logits, const int32_t* idx0, const int32_t* idx1,
                          int64_t rows, int64_t cols, const uint32_t* key_dev, int64_t dim1_size,
                          int axis, int32_t* out_pos);

/* ---- candidate-level sampler ---------------------------------------------------
 * topk_logits [rows, k] (F32 or BF16) sorted descending with masked positions equal to
 * replace_val, topk_idx [rows, k] int32.  Top-p mask on unscaled logits, divide by
 * temperature, Gumbel noise, arg-max, greedy when temperature < 1e-5.
 * Noise: `noise` (nullable) is the dense uniform tensor [*, noise_stride] read at
 * (row + dim0_offset, token); if NULL the threefry key (key0, key1) is used with
 * counter (row + dim0_offset) * vocab_size + token.
 * Replaces tallax/_src/sampling.py:185-208 (_top_p_and_sample).                     */
int tlx_top_p_and_sample(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx,
                         int64_t rows, int k, const float* top_p, const float* temperature,
                         const float* noise, int64_t noise_stride, uint32_t key0, uint32_t key1,
                         int64_t vocab_size, double replace_val, int64_t dim0_offset,
                         int32_t* out_tokens);
int tlx_top_p_and_sample_dev(void* stream, const void* topk_logits, int dtype, const int32_t* topk_idx,
                             int64_t rows, int k, const float* top_p, const float* temperature,
                             const float* noise, int64_t noise_stride, const uint32_t* key_dev,
                             int64_t vocab_size, double replace_val, const int32_t* dim0_offset_dev,
                             int32_t* out_tokens);

/* ---- fused sampler -------------------------------------------------------------
 * logits [rows, vocab] (F32 or BF16, row stride in elements) -> token ids int32[rows]
 * in one call: per-row top-k (0 or >= vocab disables it), top-p, temperature,
 * Gumbel noise (dense tensor or threefry key as above), greedy override.
 * out_status (nullable, device int32[rows]): bit 0 = the row took a path for rows without
 * (or with a very large) top-k, bit 1 = a bounded wait gave up (result invalid), bit 2 = the
 * row needed a second pass (first threshold too high, or candidate list overflow).
 * All of the call's work is ordered on `stream`.  Only after tlx_init(device,
 * TLX_INIT_SIDE_STREAM) may part of it run on a stream owned by the library, forked from
 * `stream` and joined back to it inside the call (also when a launch or an event call fails).
 * Replaces the whole of tallax/_src/sampling.py:331-343 (`sample`), i.e. the
 * top_dynamic_k kernel (top_k.py:482-506) followed by _top_p_and_sample.            */
size_t tlx_sample_workspace_bytes(int64_t rows, int64_t vocab);
int tlx_sample(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab,
               int64_t row_stride, const int32_t* top_k, const float* top_p,
               const float* temperature, const float* noise, int64_t noise_stride, uint32_t key0,
               uint32_t key1, int64_t dim0_offset, int32_t* out_tokens, int32_t* out_status,
               void* workspace, size_t workspace_bytes);
int tlx_sample_dev(void* stream, const void* logits, int dtype, int64_t rows, int64_t vocab,
                   int64_t row_stride, const int32_t* top_k, const float* top_p,
                   const float* temperature, const float* noise, int64_t noise_stride,
                   const uint32_t* key_dev, const int32_t* dim0_offset_dev, int32_t* out_tokens,
                   int32_t* out_status, void* workspace, size_t workspace_bytes);

/* ---- vocab-sharded sampler -----------------------------------------------------
 * Stage 1, on each shard: the shard's top-`k_cand` as (f32 value, GLOBAL token id =
 * local column + col_offset, uniform noise at that token), each [rows, k_cand].
 * `noise` is the shard's slice [rows, v_local] (stride in elements) or NULL for the
 * threefry key with counter (row + dim0_offset) * vocab_total + global token.
 * Stage 2, after the candidates of all shards were gathered: candidate i of row r is read
 * at (i / k_per_block) * block_stride + r * row_stride + (i % k_per_block) in each of the
 * three arrays (a plain [rows, n_cand] layout is k_per_block = row_stride = n_cand,
 * block_stride = 0; the output of an all-gather of per-shard [rows, k] blocks is
 * k_per_block = row_stride = k, block_stride = the distance between shards' blocks).
 * Blocks must be in ascending token order.  Merge by (value desc, token asc), keep
 * top_k[row] (<= 0 keeps all candidates), then the sampler tail.
 * Replaces the shard-mapped body of tallax/_src/sampling.py:305-320.                */
size_t tlx_shard_candidates_workspace_bytes(int64_t rows, int64_t v_local, int k_cand);
int tlx_shard_candidates(void* stream, const void* logits, int dtype, int64_t rows, int64_t v_local,
                         int64_t row_stride, int64_t col_offset, int k_cand, const float* noise,
                         int64_t noise_stride, uint32_t key0, uint32_t key1, int64_t vocab_total,
                         int64_t dim0_offset, float* out_vals, int32_t* out_idx, float* out_noise,
                         void* workspace, size_t workspace_bytes);
int tlx_shard_candidates_dev(void* stream, const void* logits, int dtype, int64_t rows,
                             int64_t v_local, int64_t row_stride, int64_t col_offset, int k_cand,
                             const float* noise, int64_t noise_stride, const uint32_t* key_dev,
                             int64_t vocab_total, const int32_t* dim0_offset_dev, float* out_vals,
                             int32_t* out_idx, float* out_noise, void* workspace,
                             size_t workspace_bytes);
int tlx_merge_and_sample(void* stream, const float* cand_vals, const int32_t* cand_idx,
                         const float* cand_noise, int64_t rows, int n_cand, int k_per_block,
                         int64_t block_stride, int64_t row_stride, const int32_t* top_k,
                         const float* top_p, const float* temperature, int32_t* out_tokens);

/* ---- vocab-sharded sampler, candidates exchanged over peer memory ------------------
 * The all-gather between the two stages (jax.lax.all_gather in tallax/_src/sampling.py:312-316)
 * done by the stage-1 kernel itself: every rank owns an exchange buffer (tlx_exchange_bytes, the
 * same rows, k_cand and world on every rank) and maps the other ranks' buffers; rank s stores each
 * row's candidates into slot s of every rank's buffer over NVLink and counts the row's arrival
 * there; the stage-2 kernel of a rank waits per row (bounded: two seconds, then the buffer's error
 * word and *out_status are set and the row is merged as it is) until all `world` blocks have
 * arrived.  No collective and no host synchronisation between the two calls.  Every rank makes the
 * same sequence of calls (one tlx_exchange_shard_candidates, then one
 * tlx_exchange_merge_and_sample, per step); the ranks must have finished creating and mapping
 * the buffers (a host barrier) before the first step.  After a wait gave up the buffers are out
 * of step: destroy and recreate them.  A call whose rows, k_cand or world are not those the buffer
 * was created with touches no buffer: the error word becomes 2, stage 2 sets *out_status = 2 and
 * writes token -1.
 *
 * tlx_exchange_create allocates and clears this rank's buffer (the one allocation the library makes:
 * an inter-process handle covers a whole device allocation) and writes its handle, which the other
 * processes pass to tlx_exchange_open; in one process with several devices, or to stand in for
 * several ranks on one device, plain pointers serve and no handle is needed (ipc_handle NULL).
 * `exchange_of_rank` is a HOST array of `world` device pointers, [rank] this rank's own buffer.
 * The other arguments are those of tlx_shard_candidates / _dev (key_dev NULL: key0, key1;
 * dim0_offset_dev NULL: dim0_offset) and tlx_merge_and_sample.  world <= 16.           */
#define TLX_EXCHANGE_HANDLE_BYTES 64
size_t tlx_exchange_bytes(int64_t rows, int k_cand, int world);
int tlx_exchange_create(int64_t rows, int k_cand, int world, void** exchange,
                        unsigned char* ipc_handle /* TLX_EXCHANGE_HANDLE_BYTES, or NULL */);
int tlx_exchange_open(const unsigned char* ipc_handle, void** exchange);
int tlx_exchange_close(void* exchange);      /* a buffer mapped by tlx_exchange_open */
int tlx_exchange_destroy(void* exchange);    /* a buffer made by tlx_exchange_create */
int tlx_exchange_status(void* stream, const void* exchange, uint32_t* steps, uint32_t* error);
int tlx_exchange_shard_candidates(void* stream, const void* logits, int dtype, int64_t rows,
                                  int64_t v_local, int64_t row_stride, int64_t col_offset,
                                  int k_cand, const float* noise, int64_t noise_stride,
                                  const uint32_t* key_dev, uint32_t key0, uint32_t key1,
                                  int64_t vocab_total, int64_t dim0_offset,
                                  const int32_t* dim0_offset_dev, int rank, int world,
                                  void* const* exchange_of_rank);
int tlx_exchange_merge_and_sample(void* stream, void* exchange, int64_t rows, int k_cand,
                                  int world, const int32_t* top_k, const float* top_p,
                                  const float* temperature, int32_t* out_tokens,
                                  int32_t* out_status /* nullable */);

#ifdef __cplusplus
}
#endif
#endif /* TALLAX_B200_H_ */
