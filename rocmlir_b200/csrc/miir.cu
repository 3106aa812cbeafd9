// The string-configured handle API (include/miir_b200.h), the counterpart of mlir/tools/rocmlir-lib/rocmlir-lib.cpp.
// A handle holds a parsed and validated problem; "lowering" selects the tile configuration; the "binary" is a
// launch descriptor. Like the reference (rocmlir-lib.cpp:115-119) every entry point takes one process-wide mutex,
// and nothing is printed on failure.
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/miir_b200.h"
#include "lib_state.h"
#include "problem.h"

namespace rb {
namespace {

std::mutex g_miir_mutex;

// What miirBufferGet hands out. Plain data: it can be stored and passed back on another day or process.
struct LaunchDescriptor {
  char magic[8];       // "RB2KDSC\0"
  uint32_t version;    // layout version of this struct
  uint32_t kind;
  uint32_t variant;    // tile configuration (rbSetGemmVariant word), 0 for attention
  uint32_t workspace;  // bytes
  RbConvProblem conv;
  RbGemmProblem gemm;
  RbAttentionProblem att;   // bias / mask / scale tensor pointers are always NULL in a descriptor
};
constexpr char kMagic[8] = {'R', 'B', '2', 'K', 'D', 'S', 'C', '\0'};
constexpr uint32_t kDescVersion = 1;

struct Handle {
  LaunchDescriptor d;
  ProblemDesc desc;
  bool tuned = false, binary = false;
  size_t grid = 0, block = 0;
};

MiirStatus lower(Handle* h, bool binary) {
  if (!h) return MIIR_INVALID_PARAM;
  RbGemmProblem gp;
  bool have_gemm = false;
  if (h->d.kind == kConv) {
    if (rbConvGetGemmProblem(&h->d.conv, &gp) != RB_SUCCESS) return MIIR_BUILD_FAILURE;
    have_gemm = true;
  } else if (h->d.kind == kGemm) {
    gp = h->d.gemm;
    have_gemm = true;
  }
  if (have_gemm) {
    const int saved_variant = rbGetGemmVariant();
    rbSetGemmVariant((int)h->d.variant);
    RbGemmConfigInfo info;
    const RbStatus st = rbGemmGetConfig(&gp, &info);
    rbSetGemmVariant(saved_variant);
    if (st != RB_SUCCESS) return MIIR_BUILD_FAILURE;
    h->grid = info.grid;
    h->block = info.block;
  } else {
    // attention: one CTA per pair of 128-row query tiles (single tiles for short sequences), 10 or 8 warps
    const RbAttentionProblem& a = h->d.att;
    const long long tiles = (a.seq_q + 127) / 128;
    const bool two = a.seq_q > 128 && (a.has_scale ? a.scale : 1.0f) >= 0.0f;   // the same rule as the launch
    h->grid = (size_t)((long long)a.g * (two ? (tiles + 1) / 2 : tiles));
    h->block = two ? 384 : 256;
  }
  h->tuned = true;
  if (binary) h->binary = true;
  return MIIR_SUCCESS;
}

MiirStatus launch_descriptor(const LaunchDescriptor& d, void* a0, void* a1, void* a2, void* extra, void* ws,
                             size_t ws_bytes, void* stream) {
  RbStatus st = RB_INVALID_PARAM;
  if (d.kind == kConv) {
    const int saved_variant = rbGetGemmVariant();
    rbSetGemmVariant((int)d.variant);
    st = rbConv(&d.conv, a0, a1, a2, ws, ws_bytes, stream);
    rbSetGemmVariant(saved_variant);
  } else if (d.kind == kGemm) {
    const int saved_variant = rbGetGemmVariant();
    rbSetGemmVariant((int)d.variant);
    st = rbGemm(&d.gemm, nullptr, a0, a1, a2, ws, ws_bytes, stream);
    rbSetGemmVariant(saved_variant);
  } else if (d.kind == kAttention) {
    st = rbAttention(&d.att, a0, a1, a2, extra, stream);
  }
  if (st == RB_SUCCESS) return MIIR_SUCCESS;
  return (st == RB_INVALID_PARAM || st == RB_WORKSPACE_TOO_SMALL) ? MIIR_INVALID_PARAM : MIIR_BUILD_FAILURE;
}

}  // namespace
}  // namespace rb

using namespace rb;

extern "C" MiirHandle miirCreateHandle(const char* options) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  Handle* h = new Handle;
  if (!parse_problem(options, &h->desc) || h->desc.kernel_id > 0 /* one handle is the whole operation */ ||
      h->desc.workspace > 0x7fffffffu /* the reference's workspace size is an int */) {
    delete h;
    return nullptr;
  }
  memset(&h->d, 0, sizeof(h->d));
  memcpy(h->d.magic, kMagic, 8);
  h->d.version = kDescVersion;
  h->d.kind = h->desc.kind;
  h->d.variant = h->desc.variant;
  h->d.workspace = (uint32_t)h->desc.workspace;
  h->d.conv = h->desc.conv;
  h->d.gemm = h->desc.gemm;
  h->d.att = h->desc.att;
  return h;
}

extern "C" int miirGetKernelCount(MiirHandle handle) { return handle ? 1 : -1; }

extern "C" int miirGetWorkspaceSize(MiirHandle handle) {
  return handle ? (int)static_cast<Handle*>(handle)->d.workspace : 0;
}

extern "C" MiirStatus miirLowerTuningParams(MiirHandle handle) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  return lower(static_cast<Handle*>(handle), false);
}

extern "C" MiirStatus miirLowerBin(MiirHandle handle) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  return lower(static_cast<Handle*>(handle), true);
}

extern "C" MiirStatus miirBufferGet(MiirHandle handle, char* buffer, size_t* size) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  if (!buffer && !size) return MIIR_INVALID_PARAM;
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return MIIR_INVALID_PARAM;
  if (!h->binary) return MIIR_INVALID_MODULE;
  if (h->d.kind == kAttention) return MIIR_BUILD_FAILURE;   // the attention kernels are not part of the cubin image
  const void* image = nullptr;
  size_t bytes = 0;
  if (rbGetKernelBinary(&image, &bytes) != RB_SUCCESS) return MIIR_BUILD_FAILURE;
  if (buffer) memcpy(buffer, image, bytes);
  if (size) *size = bytes;
  return MIIR_SUCCESS;
}

extern "C" MiirStatus miirDescriptorGet(MiirHandle handle, char* buffer, size_t* size) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  if (!buffer && !size) return MIIR_INVALID_PARAM;
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return MIIR_INVALID_PARAM;
  if (!h->binary) return MIIR_INVALID_MODULE;
  if (!buffer) {
    *size = sizeof(LaunchDescriptor);
  } else {
    memcpy(buffer, &h->d, sizeof(LaunchDescriptor));
    if (size) *size = sizeof(LaunchDescriptor);
  }
  return MIIR_SUCCESS;
}

extern "C" MiirStatus miirGetKernelLaunch(MiirHandle handle, void* arg0, void* arg1, void* arg2, RbKernelLaunch* out) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || !out) return MIIR_INVALID_PARAM;
  LaunchDescriptor d;
  {
    const std::lock_guard<std::mutex> lock(g_miir_mutex);
    if (!h->binary) return MIIR_INVALID_MODULE;
    d = h->d;
  }
  RbStatus st = RB_UNSUPPORTED;
  const int saved_variant = rbGetGemmVariant();
  rbSetGemmVariant((int)d.variant);
  if (d.kind == kConv) st = rbConvEncodeLaunch(&d.conv, nullptr, -1, arg0, arg1, arg2, out);
  else if (d.kind == kGemm) st = rbGemmEncodeLaunch(&d.gemm, nullptr, arg0, arg1, arg2, out);
  rbSetGemmVariant(saved_variant);
  if (st == RB_SUCCESS) return MIIR_SUCCESS;
  return st == RB_INVALID_PARAM ? MIIR_INVALID_PARAM : MIIR_BUILD_FAILURE;
}

extern "C" MiirStatus miirGetExecutionDims(MiirHandle handle, size_t* global_size, size_t* local_size) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  if (!global_size || !local_size) return MIIR_INVALID_PARAM;
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return MIIR_INVALID_PARAM;
  if (!h->tuned) return MIIR_INVALID_MODULE;
  *global_size = h->grid * h->block;
  *local_size = h->block;
  return MIIR_SUCCESS;
}

extern "C" MiirStatus miirDestroyHandle(MiirHandle handle) {
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  if (!handle) return MIIR_INVALID_PARAM;
  delete static_cast<Handle*>(handle);
  return MIIR_SUCCESS;
}

extern "C" MiirStatus miirGetArgSizes(MiirHandle handle, size_t* sizes) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h || !sizes) return MIIR_INVALID_PARAM;
  const std::lock_guard<std::mutex> lock(g_miir_mutex);
  sizes[0] = sizes[1] = sizes[2] = sizes[3] = 0;
  if (h->d.kind == kConv) {
    const RbConvProblem& c = h->d.conv;
    const size_t es = dtype_bytes(c.data_type);
    const size_t es_o = c.data_type == RB_I8 ? 4 : (c.data_type == RB_F8E4M3 || c.data_type == RB_F8E5M2) ? 4 : es;
    sizes[0] = (size_t)c.g * c.k * c.c * c.y * c.x * es;                 // c and k count channels per group
    sizes[1] = (size_t)c.n * c.g * c.c * c.h * c.w * es;
    sizes[2] = (size_t)c.n * c.g * c.k * c.ho * c.wo * (c.direction == 0 ? es_o : es);
  } else if (h->d.kind == kGemm) {
    const RbGemmProblem& g = h->d.gemm;
    sizes[0] = (size_t)g.g * g.m * g.k * dtype_bytes(g.ab_type);
    sizes[1] = (size_t)g.g * g.k * g.n * dtype_bytes(g.ab_type);
    sizes[2] = (size_t)g.g * g.m * g.n * dtype_bytes(g.c_type);
  } else if (h->d.kind == kAttention) {
    const RbAttentionProblem& a = h->d.att;
    const size_t es = dtype_bytes(a.data_type), es_v = a.data_type == RB_I8 ? 2 : es;
    sizes[0] = (size_t)a.g * a.seq_q * a.head_qk * es;
    sizes[1] = (size_t)a.g * a.seq_k * a.head_qk * es;
    sizes[2] = (size_t)a.g * a.seq_k * a.head_v * es_v;
    sizes[3] = (size_t)a.g * a.seq_q * a.head_v * es_v;
  } else {
    return MIIR_INVALID_MODULE;
  }
  return MIIR_SUCCESS;
}

extern "C" MiirStatus miirLaunch(MiirHandle handle, void* arg0, void* arg1, void* arg2, void* extra, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  Handle* h = static_cast<Handle*>(handle);
  if (!h) return MIIR_INVALID_PARAM;
  LaunchDescriptor d;
  {
    const std::lock_guard<std::mutex> lock(g_miir_mutex);
    if (!h->tuned) return MIIR_INVALID_MODULE;
    d = h->d;
  }
  return launch_descriptor(d, arg0, arg1, arg2, extra, workspace, workspace_bytes, stream);
}

extern "C" MiirStatus miirLaunchFromBuffer(const char* buffer, size_t size, void* arg0, void* arg1, void* arg2,
                                           void* extra, void* workspace, size_t workspace_bytes, void* stream) {
  if (!buffer || size != sizeof(LaunchDescriptor)) return MIIR_INVALID_PARAM;
  LaunchDescriptor d;
  memcpy(&d, buffer, sizeof(d));
  if (memcmp(d.magic, kMagic, 8) != 0 || d.version != kDescVersion) return MIIR_INVALID_MODULE;
  d.att.bias = nullptr;
  d.att.mask = nullptr;
  d.att.scale_tensor = nullptr;
  return launch_descriptor(d, arg0, arg1, arg2, extra, workspace, workspace_bytes, stream);
}
