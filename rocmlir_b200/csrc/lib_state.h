// Process-wide state of the library shared by its translation units: error text, launch counter,
// the device status word, and the driver entry point used to encode TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/rocmlir_b200.h"

namespace rb {

// Sets the thread's last-error text and returns `st`.
RbStatus fail(RbStatus st, const std::string& msg);
void count_launch(int n = 1);

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  uint32_t* status_word = nullptr;  // device address of the status word
};
// Per-device lazy initialisation (current device). Returns nullptr and sets the error on failure.
const DeviceInfo* device_info();

// Encodes a rank-`rank` tiled tensor map (128-byte swizzle unless `swizzle` says otherwise).
// dims/box are innermost-first; strides_bytes has rank-1 entries (dimension 1 upward).
bool encode_tiled(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                  std::string* err);

inline size_t dtype_bytes(int t) {
  switch (t) {
    case RB_F32: case RB_I32: return 4;
    case RB_F16: case RB_BF16: return 2;
    case RB_I8: case RB_F8E4M3: return 1;
    default: return 0;
  }
}

#define RB_CUDA_TRY(expr)                                                                          \
  do {                                                                                             \
    cudaError_t e_ = (expr);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      return ::rb::fail(RB_CUDA_ERROR, std::string(#expr) + ": " + cudaGetErrorString(e_));       \
  } while (0)

}  // namespace rb
