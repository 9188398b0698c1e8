// Exchange buffers of the vocab-sharded sampler: allocation, inter-process mapping, status.
// The kernels that use them are the candidate kernels (topk.cu) and the merge kernel (sampler.cu).
#include "exchange.cuh"
#include "tlx_common.cuh"

#include <cstring>

using namespace tlx;

extern "C" {

size_t tlx_exchange_bytes(int64_t rows, int k_cand, int world) {
  if (rows < 1 || k_cand < 1 || world < 1 || world > kExchangeMaxWorld) return 0;
  return exchange_layout(rows, k_cand, world).bytes;
}

int tlx_exchange_create(int64_t rows, int k_cand, int world, void** exchange, unsigned char* ipc_handle) {
  TLX_CHECK_ARG(exchange, "exchange_create: null pointer");
  const size_t bytes = tlx_exchange_bytes(rows, k_cand, world);
  TLX_CHECK_ARG(bytes > 0, "exchange_create: bad extent (rows %lld, k %d, world %d)", (long long)rows, k_cand, world);
  void* buf = nullptr;
  cudaError_t e = cudaMalloc(&buf, bytes);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "exchange_create: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  e = cudaMemset(buf, 0, bytes);
  if (e == cudaSuccess) {
    ExchangeHeader h{};
    h.rows = (uint32_t)rows;
    h.k_cand = (uint32_t)k_cand;
    h.world = (uint32_t)world;
    e = cudaMemcpy(buf, &h, sizeof(h), cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && ipc_handle) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, buf);
    if (e == cudaSuccess) {
      static_assert(sizeof(h) == TLX_EXCHANGE_HANDLE_BYTES, "handle size");
      memcpy(ipc_handle, &h, sizeof(h));
    }
  }
  if (e != cudaSuccess) {
    cudaFree(buf);
    return set_error(TLX_ERR_CUDA, "exchange_create: %s", cudaGetErrorString(e));
  }
  *exchange = buf;
  return TLX_OK;
}

int tlx_exchange_open(const unsigned char* ipc_handle, void** exchange) {
  TLX_CHECK_ARG(ipc_handle && exchange, "exchange_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  void* buf = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&buf, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "exchange_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *exchange = buf;
  return TLX_OK;
}

int tlx_exchange_close(void* exchange) {
  if (!exchange) return TLX_OK;
  cudaError_t e = cudaIpcCloseMemHandle(exchange);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "exchange_close: %s", cudaGetErrorString(e));
  return TLX_OK;
}

int tlx_exchange_destroy(void* exchange) {
  if (!exchange) return TLX_OK;
  cudaError_t e = cudaFree(exchange);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "exchange_destroy: %s", cudaGetErrorString(e));
  return TLX_OK;
}

int tlx_exchange_status(void* stream, const void* exchange, uint32_t* steps, uint32_t* error) {
  TLX_CHECK_ARG(exchange, "exchange_status: null pointer");
  ExchangeHeader h;
  cudaError_t e = cudaMemcpyAsync(&h, exchange, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return set_error(TLX_ERR_CUDA, "exchange_status: %s", cudaGetErrorString(e));
  if (steps) *steps = h.step;
  if (error) *error = h.error;
  return TLX_OK;
}

}  // extern "C"
