// Host-buffer entry points: the counterpart of the `<kernel>_gpu` wrapper that rocmlir-gen's host
// harness emits around a kernel (gpu.alloc, memcpy in, launch, memcpy out;
// mlir/tools/rocmlir-gen/rocmlir-gen.cpp:1211-1283). Device staging memory is a grow-only arena owned
// by the calling thread, so repeated calls of the same size allocate nothing.
#include <cuda_runtime.h>

#include "lib_state.h"

namespace rb {
namespace {
struct Arena {
  void* ptr = nullptr;
  size_t size = 0;
  int device = -1;
};
thread_local Arena t_arena;

RbStatus arena_reserve(size_t bytes) {
  int dev = 0;
  RB_CUDA_TRY(cudaGetDevice(&dev));
  if (t_arena.device == dev && t_arena.size >= bytes) return RB_SUCCESS;
  if (t_arena.ptr) {
    RB_CUDA_TRY(cudaDeviceSynchronize());
    RB_CUDA_TRY(cudaFree(t_arena.ptr));
    t_arena = Arena();
  }
  RB_CUDA_TRY(cudaMalloc(&t_arena.ptr, bytes));
  t_arena.size = bytes;
  t_arena.device = dev;
  return RB_SUCCESS;
}
size_t up256(size_t x) { return (x + 255) / 256 * 256; }
}  // namespace
}  // namespace rb

using namespace rb;

extern "C" RbStatus rbGemmHost(const RbGemmProblem* p, const RbEpilogue* epi_host, const void* a_host,
                               const void* b_host, void* c_host, void* stream_v) {
  if (!p || !a_host || !b_host || !c_host) return fail(RB_INVALID_PARAM, "NULL argument");
  if (p->g <= 0 || p->m <= 0 || p->n <= 0 || p->k <= 0) return fail(RB_INVALID_PARAM, "g, m, n, k must be positive");
  const size_t es = dtype_bytes(p->ab_type), es_c = dtype_bytes(p->c_type);
  if (!es || !es_c) return fail(RB_INVALID_PARAM, "unknown element type");
  if (!device_info()) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const size_t a_bytes = (size_t)p->g * p->m * p->k * es, b_bytes = (size_t)p->g * p->k * p->n * es;
  const size_t c_bytes = (size_t)p->g * p->m * p->n * es_c;
  const size_t ws_bytes = rbGemmWorkspaceSize(p);
  const uint32_t flags = epi_host ? epi_host->flags : 0u;
  if (flags & (RB_EPI_RESIDUAL | RB_EPI_BIAS_ROW | RB_EPI_BIAS_SCALAR))
    return fail(RB_UNSUPPORTED, "the host-buffer entry point carries per-column epilogue vectors only");
  if (p->store_method != 0) return fail(RB_UNSUPPORTED, "the host-buffer entry point computes C = A.B only");
  const size_t scale_bytes = (flags & RB_EPI_COL_SCALE) ? (size_t)p->n * 4 : 0;
  const size_t bias_bytes = (flags & RB_EPI_BIAS) ? (size_t)p->n * dtype_bytes(epi_host->bias_type) : 0;
  const size_t total = up256(a_bytes) + up256(b_bytes) + up256(c_bytes) + up256(ws_bytes) + up256(scale_bytes) +
                       up256(bias_bytes);
  RbStatus st = arena_reserve(total);
  if (st != RB_SUCCESS) return st;
  uint8_t* base = static_cast<uint8_t*>(t_arena.ptr);
  uint8_t* da = base;
  uint8_t* db = da + up256(a_bytes);
  uint8_t* dc = db + up256(b_bytes);
  uint8_t* dws = dc + up256(c_bytes);
  uint8_t* dscale = dws + up256(ws_bytes);
  uint8_t* dbias = dscale + up256(scale_bytes);
  RB_CUDA_TRY(cudaMemcpyAsync(da, a_host, a_bytes, cudaMemcpyHostToDevice, stream));
  RB_CUDA_TRY(cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, stream));
  RbEpilogue e;
  if (epi_host) {
    e = *epi_host;
    if (scale_bytes) {
      if (!epi_host->col_scale) return fail(RB_INVALID_PARAM, "col_scale is NULL");
      RB_CUDA_TRY(cudaMemcpyAsync(dscale, epi_host->col_scale, scale_bytes, cudaMemcpyHostToDevice, stream));
      e.col_scale = reinterpret_cast<const float*>(dscale);
    }
    if (bias_bytes) {
      if (!epi_host->bias) return fail(RB_INVALID_PARAM, "bias is NULL");
      RB_CUDA_TRY(cudaMemcpyAsync(dbias, epi_host->bias, bias_bytes, cudaMemcpyHostToDevice, stream));
      e.bias = dbias;
    }
  }
  st = rbGemm(p, epi_host ? &e : nullptr, da, db, dc, ws_bytes ? dws : nullptr, ws_bytes, stream_v);
  if (st != RB_SUCCESS) return st;
  RB_CUDA_TRY(cudaMemcpyAsync(c_host, dc, c_bytes, cudaMemcpyDeviceToHost, stream));
  RB_CUDA_TRY(cudaStreamSynchronize(stream));
  // This entry point is synchronous, so it can report what the asynchronous ones leave to rbReadKernelStatus: a
  // bounded device-side wait that ran out (the result in c_host is then not valid).
  uint32_t word = 0;
  st = read_status_word(&word, true);
  if (st != RB_SUCCESS) return st;
  if (word) return fail(RB_KERNEL_TIMEOUT, "a bounded device-side wait ran out (status code " + std::to_string(word) + ")");
  return RB_SUCCESS;
}
