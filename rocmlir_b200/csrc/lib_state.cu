#include "lib_state.h"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace rb {

namespace {
thread_local std::string t_last_error;
thread_local unsigned long long* t_trace = nullptr;
thread_local size_t t_trace_len = 0;
std::atomic<uint64_t> g_launches{0};
__device__ uint32_t g_status_word;  // written by kernels whose bounded waits run out

constexpr int kMaxDevices = 16;
DeviceInfo g_devices[kMaxDevices];
std::once_flag g_device_once[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_encode_im2col_once;
}  // namespace

RbStatus fail(RbStatus st, const std::string& msg) {
  t_last_error = msg;
  return st;
}

unsigned long long* trace_buffer(size_t need_u64) { return (t_trace && t_trace_len >= need_u64) ? t_trace : nullptr; }

RbStatus ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> granted;   // largest size set so far
  int dev = 0;
  RB_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  int& have = granted[std::make_pair(dev, kernel)];
  if (bytes <= have) return RB_SUCCESS;
  RB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  have = bytes;
  return RB_SUCCESS;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

const DeviceInfo* device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(RB_CUDA_ERROR, "no usable CUDA device (the library has no CPU path)");
    return nullptr;
  }
  std::call_once(g_device_once[dev], [dev] {
    DeviceInfo d;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return;
    if (prop.major != 10) return;  // sm_100a kernels only
    d.sm_count = prop.multiProcessorCount;
    d.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return;
    d.status_word = static_cast<uint32_t*>(p);
    if (cudaMemset(p, 0, sizeof(uint32_t)) != cudaSuccess) return;
    d.device = dev;
    g_devices[dev] = d;
  });
  if (g_devices[dev].device != dev) {
    fail(RB_CUDA_ERROR, "device is not an sm_100 GPU or could not be initialised");
    return nullptr;
  }
  return &g_devices[dev];
}

int planning_sm_count() {
  static const int cached = [] {
    int dev = 0, n = 0, major = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess && major == 10 &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      return n;
    (void)cudaGetLastError();   // no device: not an error for a planning query
    return 148;
  }();
  return cached;
}

RbStatus read_status_word(uint32_t* out, bool clear) {
  const DeviceInfo* d = device_info();
  if (!d) return RB_CUDA_ERROR;
  RB_CUDA_TRY(cudaMemcpy(out, d->status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (clear && *out) RB_CUDA_TRY(cudaMemset(d->status_word, 0, sizeof(uint32_t)));
  return RB_SUCCESS;
}

bool encode_tiled(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle, std::string* err) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_encode) {
    if (err) *err = "cuTensorMapEncodeTiled is not available from the driver";
    return false;
  }
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) {
      *err = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r) + " (dims";
      for (int i = 0; i < rank; ++i) *err += " " + std::to_string(dims[i]);
      *err += "; strides";
      for (int i = 0; i + 1 < rank; ++i) *err += " " + std::to_string(strides_bytes[i]);
      *err += "; box";
      for (int i = 0; i < rank; ++i) *err += " " + std::to_string(box[i]);
      *err += ")";
    }
    return false;
  }
  return true;
}

bool encode_im2col_nhwc(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[4],
                        const uint64_t strides_bytes[3], const int lower_corner[2], const int upper_corner[2],
                        uint32_t channels_per_pixel, uint32_t pixels_per_column, const uint32_t traversal_stride[2],
                        std::string* err) {
  std::call_once(g_encode_im2col_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  });
  if (!g_encode_im2col) {
    if (err) *err = "cuTensorMapEncodeIm2col is not available from the driver";
    return false;
  }
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t s[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t es[4] = {1, traversal_stride[0], traversal_stride[1], 1};
  CUresult r = g_encode_im2col(out, dt, 4, const_cast<void*>(base), d, s, lower_corner, upper_corner,
                               channels_per_pixel, pixels_per_column, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err)
      *err = "cuTensorMapEncodeIm2col failed with CUresult " + std::to_string((int)r) + " (corners " +
             std::to_string(lower_corner[0]) + "," + std::to_string(lower_corner[1]) + " / " +
             std::to_string(upper_corner[0]) + "," + std::to_string(upper_corner[1]) + ")";
    return false;
  }
  return true;
}

}  // namespace rb

extern "C" {

RbStatus rbReadKernelStatus(uint32_t* status_out, int clear) {
  const rb::DeviceInfo* d = rb::device_info();
  if (!d) return RB_CUDA_ERROR;
  if (!status_out) return rb::fail(RB_INVALID_PARAM, "status_out is NULL");
  RB_CUDA_TRY(cudaDeviceSynchronize());
  RB_CUDA_TRY(cudaMemcpy(status_out, d->status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (clear) RB_CUDA_TRY(cudaMemset(d->status_word, 0, sizeof(uint32_t)));
  return RB_SUCCESS;
}

void rbSetTraceBuffer(unsigned long long* device_buf, size_t n_u64) {
  rb::t_trace = device_buf;
  rb::t_trace_len = n_u64;
}

uint64_t rbLaunchCount(void) { return rb::g_launches.load(std::memory_order_relaxed); }

const char* rbGetLastError(void) { return rb::t_last_error.c_str(); }

}  // extern "C"
