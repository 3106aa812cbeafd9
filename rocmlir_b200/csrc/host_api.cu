// Host-buffer entry points: the counterpart of the `<kernel>_gpu` wrapper that rocmlir-gen's host
// harness emits around a kernel (gpu.alloc, memcpy in, launch, memcpy out;
// mlir/tools/rocmlir-gen/rocmlir-gen.cpp:1211-1283). Device staging memory is a grow-only arena owned
// by the calling thread, so repeated calls of the same size allocate nothing.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

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

// Copy streams and events of the pipelined host path, one set per calling thread and device, created on first use
// and kept for the life of the thread.
struct HostPipe {
  static constexpr int kEvents = 16;
  int device = -1;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, ev[kEvents] = {}, evg[kEvents] = {};
};
thread_local HostPipe t_pipe;

HostPipe* host_pipe() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { fail(RB_CUDA_ERROR, "cudaGetDevice failed"); return nullptr; }
  if (t_pipe.device == dev) return &t_pipe;
  HostPipe hp;
  bool ok = cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking) == cudaSuccess &&
            cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking) == cudaSuccess &&
            cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < HostPipe::kEvents; ++i)
    ok = cudaEventCreateWithFlags(&hp.ev[i], cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&hp.evg[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) { fail(RB_CUDA_ERROR, "could not create the copy streams of the host path"); return nullptr; }
  hp.device = dev;
  t_pipe = hp;
  return &t_pipe;
}
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
  // Pipelined form: B first, then A in blocks of rows; the GEMM of a block runs as soon as its rows have arrived and
  // its rows of C travel back while later blocks are still uploading, so both directions of the host link are busy at
  // once. Rows of C depend on their own rows of A only and every element keeps its K order, so the result is bit for
  // bit that of one rbGemm over the whole problem. Applies to one group with A and C stored row by row.
  // rows per block: 1024 by default (measured at 4096^3 f16 over PCIe gen5: 512 rows 80.0, 1024 rows 85.4 TFLOP/s end
  // to end); RB_HOST_BLOCK_ROWS (a multiple of 128, read once) overrides it for experiments
  static const int kBlockRows = [] {
    const char* e = getenv("RB_HOST_BLOCK_ROWS");
    const int v = e ? atoi(e) : 0;
    return (v >= 128 && v % 128 == 0) ? v : 1024;
  }();
  const bool pipelined = p->g == 1 && !p->trans_a && !p->trans_c && p->m >= 4 * kBlockRows && ws_bytes == 0 &&
                         a_bytes + b_bytes + c_bytes >= ((size_t)8 << 20);
  if (pipelined) {
    HostPipe* hp = host_pipe();
    if (!hp) return RB_CUDA_ERROR;
    const int nblk = (p->m + kBlockRows - 1) / kBlockRows;
    RB_CUDA_TRY(cudaEventRecord(hp->start, stream));               // epilogue vectors, and whatever `stream` held before
    RB_CUDA_TRY(cudaStreamWaitEvent(hp->in, hp->start, 0));
    RB_CUDA_TRY(cudaStreamWaitEvent(hp->out, hp->start, 0));
    RB_CUDA_TRY(cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, hp->in));
    const int saved_variant = rbGetGemmVariant();
    // whole tiles per block: a K split would only add a reduction pass to a GEMM that hides behind the copies anyway
    rbSetGemmVariant((saved_variant & ~0xFF0000) | (1 << 16));
    RbStatus bst = RB_SUCCESS;
    for (int i = 0; i < nblk && bst == RB_SUCCESS; ++i) {
      const int r0 = i * kBlockRows, rows = std::min(kBlockRows, p->m - r0);
      const size_t a_off = (size_t)r0 * p->k * es, c_off = (size_t)r0 * p->n * es_c;
      cudaEvent_t ev = hp->ev[i % HostPipe::kEvents];
      cudaError_t ce = cudaMemcpyAsync(da + a_off, static_cast<const uint8_t*>(a_host) + a_off, (size_t)rows * p->k * es,
                                       cudaMemcpyHostToDevice, hp->in);
      if (ce == cudaSuccess) ce = cudaEventRecord(ev, hp->in);
      if (ce == cudaSuccess) ce = cudaStreamWaitEvent(stream, ev, 0);
      if (ce != cudaSuccess) { bst = fail(RB_CUDA_ERROR, cudaGetErrorString(ce)); break; }
      RbGemmProblem bp = *p;
      bp.m = rows;
      bst = rbGemm(&bp, epi_host ? &e : nullptr, da + a_off, db, dc + c_off, nullptr, 0, stream_v);
      if (bst != RB_SUCCESS) break;
      cudaEvent_t evg = hp->evg[i % HostPipe::kEvents];
      ce = cudaEventRecord(evg, stream);
      if (ce == cudaSuccess) ce = cudaStreamWaitEvent(hp->out, evg, 0);
      if (ce == cudaSuccess)
        ce = cudaMemcpyAsync(static_cast<uint8_t*>(c_host) + c_off, dc + c_off, (size_t)rows * p->n * es_c,
                             cudaMemcpyDeviceToHost, hp->out);
      if (ce != cudaSuccess) bst = fail(RB_CUDA_ERROR, cudaGetErrorString(ce));
    }
    rbSetGemmVariant(saved_variant);
    // the copy streams are the library's own: always drain them, also after an error
    const cudaError_t s1 = cudaStreamSynchronize(hp->in), s2 = cudaStreamSynchronize(hp->out),
                      s3 = cudaStreamSynchronize(stream);
    if (bst != RB_SUCCESS) return bst;
    RB_CUDA_TRY(s1);
    RB_CUDA_TRY(s2);
    RB_CUDA_TRY(s3);
  } else {
    RB_CUDA_TRY(cudaMemcpyAsync(da, a_host, a_bytes, cudaMemcpyHostToDevice, stream));
    RB_CUDA_TRY(cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, stream));
    st = rbGemm(p, epi_host ? &e : nullptr, da, db, dc, ws_bytes ? dws : nullptr, ws_bytes, stream_v);
    if (st != RB_SUCCESS) return st;
    RB_CUDA_TRY(cudaMemcpyAsync(c_host, dc, c_bytes, cudaMemcpyDeviceToHost, stream));
    RB_CUDA_TRY(cudaStreamSynchronize(stream));
  }
  // This entry point is synchronous, so it can report what the asynchronous ones leave to rbReadKernelStatus: a
  // bounded device-side wait that ran out (the result in c_host is then not valid).
  uint32_t word = 0;
  st = read_status_word(&word, true);
  if (st != RB_SUCCESS) return st;
  if (word) return fail(RB_KERNEL_TIMEOUT, "a bounded device-side wait ran out (status code " + std::to_string(word) + ")");
  return RB_SUCCESS;
}
