// XLA FFI handlers over the C ABI of libtallax_b200.so: what a JAX build registers with
// jax.ffi.register_ffi_target in place of the pl.pallas_call sites of tallax/_src/sampling.py:185-208 and
// :331-343, tallax/_src/sparse_random.py:43-94 and the shard-mapped body of sampling.py:305-320.
//
// Everything a handler receives under jit is a device buffer: the PRNG key (jax.random.key_data, u32[2])
// and the batch offset (axis_index * local_rows, an s32 scalar computed inside shard_map) included.  The
// handlers therefore bind the *_dev entry points, which read both on the device.
//
// Build (a maintainer with JAX installed; this translation unit is not part of the library itself):
//   g++ -shared -fPIC -std=c++17 -I$(python -c "import jax; print(jax.ffi.include_dir())") -Iinclude \
//       -I/usr/local/cuda/include tallax_b200/ffi/xla_ffi_adapter.cc -Ltallax_b200/lib -ltallax_b200 \
//       -o libtallax_b200_ffi.so
// Without the XLA headers the file compiles to an empty object, so that it can sit in the tree of a
// build that has no JAX.
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define TLX_HAVE_XLA_FFI 1
#endif
#endif

#ifdef TLX_HAVE_XLA_FFI
#include <cuda_runtime_api.h>

#include "tallax_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error as_error(int rc) {
  if (rc == TLX_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = rc == TLX_ERR_INVALID       ? ffi::ErrorCode::kInvalidArgument
                              : rc == TLX_ERR_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented
                              : rc == TLX_ERR_WORKSPACE   ? ffi::ErrorCode::kResourceExhausted
                                                          : ffi::ErrorCode::kInternal;
  return ffi::Error(code, tlx_last_error());
}

int dtype_of(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: return TLX_F32;
    case ffi::DataType::BF16: return TLX_BF16;
    case ffi::DataType::F16: return TLX_F16;
    default: return -1;
  }
}

// sample(rng_key, logits, metadata): tallax/_src/sampling.py:331-343.
// Operands: logits [rows, vocab], top_k s32[rows], top_p f32[rows], temperature f32[rows], key u32[2],
// dim0_offset s32[] ; results: tokens s32[rows], workspace u8[tlx_sample_workspace_bytes(rows, vocab)].
ffi::Error SampleImpl(cudaStream_t stream, ffi::AnyBuffer logits, ffi::Buffer<ffi::DataType::S32> top_k,
                      ffi::Buffer<ffi::DataType::F32> top_p, ffi::Buffer<ffi::DataType::F32> temperature,
                      ffi::Buffer<ffi::DataType::U32> key, ffi::Buffer<ffi::DataType::S32> dim0_offset,
                      ffi::Result<ffi::Buffer<ffi::DataType::S32>> tokens,
                      ffi::Result<ffi::Buffer<ffi::DataType::U8>> workspace) {
  const auto d = logits.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "Only 2D inputs supported");
  return as_error(tlx_sample_dev(stream, logits.untyped_data(), dtype_of(logits.element_type()), d[0], d[1], d[1],
                                 top_k.typed_data(), top_p.typed_data(), temperature.typed_data(), /*noise=*/nullptr, 0,
                                 key.typed_data(), dim0_offset.typed_data(), tokens->typed_data(), /*status=*/nullptr,
                                 workspace->typed_data(), workspace->element_count()));
}

// _top_p_and_sample: tallax/_src/sampling.py:185-208.
ffi::Error TopPAndSampleImpl(cudaStream_t stream, ffi::AnyBuffer topk_logits, ffi::Buffer<ffi::DataType::S32> topk_idx,
                             ffi::Buffer<ffi::DataType::F32> top_p, ffi::Buffer<ffi::DataType::F32> temperature,
                             ffi::Buffer<ffi::DataType::U32> key, ffi::Buffer<ffi::DataType::S32> dim0_offset,
                             int64_t vocab_size, double replace_val, ffi::Result<ffi::Buffer<ffi::DataType::S32>> tokens) {
  const auto d = topk_logits.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "Only 2D inputs supported");
  return as_error(tlx_top_p_and_sample_dev(stream, topk_logits.untyped_data(), dtype_of(topk_logits.element_type()),
                                           topk_idx.typed_data(), d[0], (int)d[1], top_p.typed_data(),
                                           temperature.typed_data(), /*noise=*/nullptr, 0, key.typed_data(), vocab_size,
                                           replace_val, dim0_offset.typed_data(), tokens->typed_data()));
}

// sparse_random_uniform: tallax/_src/sparse_random.py:43-64.
ffi::Error SparseRandomUniformImpl(cudaStream_t stream, ffi::Buffer<ffi::DataType::U32> key,
                                   ffi::Buffer<ffi::DataType::S32> idx0, ffi::Buffer<ffi::DataType::S32> idx1,
                                   int64_t dim1_size, float minval, float maxval,
                                   ffi::Result<ffi::Buffer<ffi::DataType::F32>> out) {
  return as_error(tlx_sparse_random_uniform_dev(stream, key.typed_data(), idx0.typed_data(), idx1.typed_data(),
                                                (int64_t)idx0.element_count(), dim1_size, minval, maxval,
                                                out->typed_data()));
}

// sparse_random_categorical's arg-max: tallax/_src/sparse_random.py:68-94.
ffi::Error GumbelArgmaxImpl(cudaStream_t stream, ffi::Buffer<ffi::DataType::U32> key,
                            ffi::Buffer<ffi::DataType::F32> logits, ffi::Buffer<ffi::DataType::S32> idx0,
                            ffi::Buffer<ffi::DataType::S32> idx1, int64_t dim1_size, int64_t axis,
                            ffi::Result<ffi::Buffer<ffi::DataType::S32>> pos) {
  const auto d = logits.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "Only 2D inputs supported");
  return as_error(tlx_gumbel_argmax_dev(stream, logits.typed_data(), idx0.typed_data(), idx1.typed_data(), d[0], d[1],
                                        key.typed_data(), dim1_size, (int)axis, pos->typed_data()));
}

// stage 1 of the vocab-sharded sampler (the shard-mapped body of tallax/_src/sampling.py:305-320): one
// packed result [3, rows, k_cand] f32 storage (values, global token ids, noise) ready for all_gather.
ffi::Error ShardCandidatesImpl(cudaStream_t stream, ffi::AnyBuffer logits, ffi::Buffer<ffi::DataType::U32> key,
                               ffi::Buffer<ffi::DataType::S32> dim0_offset, int64_t col_offset, int64_t k_cand,
                               int64_t vocab_total, ffi::Result<ffi::Buffer<ffi::DataType::F32>> packed) {
  const auto d = logits.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "Only 2D inputs supported");
  float* base = packed->typed_data();
  const int64_t plane = d[0] * k_cand;
  return as_error(tlx_shard_candidates_dev(stream, logits.untyped_data(), dtype_of(logits.element_type()), d[0], d[1],
                                           d[1], col_offset, (int)k_cand, /*noise=*/nullptr, 0, key.typed_data(),
                                           vocab_total, dim0_offset.typed_data(), base,
                                           reinterpret_cast<int32_t*>(base + plane), base + 2 * plane, nullptr, 0));
}

// The vocab-sharded sampler with the all_gather of tallax/_src/sampling.py:312-316 done by the kernels over
// peer memory: the exchange buffers are made and mapped at set-up (tlx_exchange_create / tlx_exchange_open on
// the host, outside jit); their device addresses reach the handlers as attributes, `exchange_of_rank` holding
// the `world` addresses in rank order.  Stage 1 has no result of its own (a dummy token keeps XLA's ordering:
// stage 2 takes it as an operand).
ffi::Error ExchangeShardCandidatesImpl(cudaStream_t stream, ffi::AnyBuffer logits, ffi::Buffer<ffi::DataType::U32> key,
                                       ffi::Buffer<ffi::DataType::S32> dim0_offset, int64_t col_offset, int64_t k_cand,
                                       int64_t vocab_total, int64_t rank, ffi::Span<const int64_t> exchange_of_rank,
                                       ffi::Result<ffi::Buffer<ffi::DataType::S32>> order_token) {
  const auto d = logits.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "Only 2D inputs supported");
  void* bufs[16];
  const int world = (int)exchange_of_rank.size();
  if (world < 1 || world > 16) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "1 to 16 ranks");
  for (int i = 0; i < world; ++i) bufs[i] = reinterpret_cast<void*>(exchange_of_rank[i]);
  (void)order_token;
  return as_error(tlx_exchange_shard_candidates(stream, logits.untyped_data(), dtype_of(logits.element_type()), d[0],
                                                d[1], d[1], col_offset, (int)k_cand, /*noise=*/nullptr, 0,
                                                key.typed_data(), 0u, 0u, vocab_total, 0, dim0_offset.typed_data(),
                                                (int)rank, world, bufs));
}

ffi::Error ExchangeMergeAndSampleImpl(cudaStream_t stream, ffi::Buffer<ffi::DataType::S32> order_token,
                                      ffi::Buffer<ffi::DataType::S32> top_k, ffi::Buffer<ffi::DataType::F32> top_p,
                                      ffi::Buffer<ffi::DataType::F32> temperature, int64_t k_cand, int64_t world,
                                      int64_t exchange, ffi::Result<ffi::Buffer<ffi::DataType::S32>> tokens,
                                      ffi::Result<ffi::Buffer<ffi::DataType::S32>> status) {
  (void)order_token;
  const int64_t rows = (int64_t)top_k.element_count();
  return as_error(tlx_exchange_merge_and_sample(stream, reinterpret_cast<void*>(exchange), rows, (int)k_cand, (int)world,
                                                top_k.typed_data(), top_p.typed_data(), temperature.typed_data(),
                                                tokens->typed_data(), status->typed_data()));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxExchangeShardCandidates, ExchangeShardCandidatesImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Attr<int64_t>("col_offset")
                                  .Attr<int64_t>("k_cand")
                                  .Attr<int64_t>("vocab_total")
                                  .Attr<int64_t>("rank")
                                  .Attr<ffi::Span<const int64_t>>("exchange_of_rank")
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxExchangeMergeAndSample, ExchangeMergeAndSampleImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Attr<int64_t>("k_cand")
                                  .Attr<int64_t>("world")
                                  .Attr<int64_t>("exchange")
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxSample, SampleImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::U8>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxTopPAndSample, TopPAndSampleImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Attr<int64_t>("vocab_size")
                                  .Attr<double>("replace_val")
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxSparseRandomUniform, SparseRandomUniformImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Attr<int64_t>("dim1_size")
                                  .Attr<float>("minval")
                                  .Attr<float>("maxval")
                                  .Ret<ffi::Buffer<ffi::DataType::F32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxGumbelArgmax, GumbelArgmaxImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Attr<int64_t>("dim1_size")
                                  .Attr<int64_t>("axis")
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(TlxShardCandidates, ShardCandidatesImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::DataType::U32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Attr<int64_t>("col_offset")
                                  .Attr<int64_t>("k_cand")
                                  .Attr<int64_t>("vocab_total")
                                  .Ret<ffi::Buffer<ffi::DataType::F32>>());
#endif  // TLX_HAVE_XLA_FFI
