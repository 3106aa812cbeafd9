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

// SM count used when planning a launch: that of the current device if it is an sm_100 GPU, else 148 (a B200).
int planning_sm_count();
// Reads the current device's status word after the caller has synchronised; nonzero = a bounded wait ran out.
// With `clear` the word is reset.
RbStatus read_status_word(uint32_t* out, bool clear);

// Encodes a rank-`rank` tiled tensor map (128-byte swizzle unless `swizzle` says otherwise).
// dims/box are innermost-first; strides_bytes has rank-1 entries (dimension 1 upward).
bool encode_tiled(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                  std::string* err);

// im2col-mode map of an NHWC tensor: dims/strides innermost-first {C, W, H, N}; box = channels x pixels.
bool encode_im2col_nhwc(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[4],
                        const uint64_t strides_bytes[3], const int lower_corner[2], const int upper_corner[2],
                        uint32_t channels_per_pixel, uint32_t pixels_per_column, const uint32_t traversal_stride[2],
                        std::string* err);

// Implicit-GEMM description of the A operand for gemm_run: the activation tensor of a convolution.
struct ConvAOperand {
  int operand = 0;           // 0: the A operand (GEMM M = N*P*Q, K = Y*X*C). 1: the B operand of a backward-weight
                             // convolution (GEMM K = N*P*Q, N = Y*X*C; B stored K x N, i.e. trans_b = 0)
  const void* tensor;        // NHWC (dense), element type = the GEMM's ab_type (f32: the hi TF32 plane)
  const void* tensor_lo = nullptr;  // f32 in accurate mode: the lo TF32 plane of the same tensor (see f32_planes)
  int N, H, W, C;            // tensor extents
  int P, Q;                  // output image (GEMM M = N * P * Q)
  int Y, X;                  // filter (GEMM K = Y * X * C)
  int stride_h, stride_w, dil_h, dil_w;
  int pad_h, pad_w;          // base pixel of output (p, q) = (p*stride_h - pad_h, q*stride_w - pad_w); may be negative pads
  int pad_h_hi, pad_w_hi;    // upper paddings (bounding box of the base pixel)
  // Result stored channel-major per image (NKHW) by the epilogue: element (row = image * c_rows_per_img + pixel, col) at
  // image * c_img_stride + col * c_col_stride + pixel. 0 = the plain [rows][cols] result.
  int c_rows_per_img = 0;
  long long c_img_stride = 0, c_col_stride = 0;
};
// rbGemm with an optional implicit operand (then `a` (or `b`) is ignored, trans_a (trans_b) must be 0, g must be 1).
// With `capture` nothing is launched: the call prepares everything as usual and writes the one kernel launch it
// would make (symbol in the library's cubin, grid, block, cluster, shared memory, parameter block) into `capture`;
// it fails with RB_UNSUPPORTED when the operation needs more than that one kernel (operand copies, a K split).
RbStatus gemm_run(const RbGemmProblem* p, const RbEpilogue* epi, const void* a, const void* b, void* c, void* workspace,
                  size_t workspace_bytes, void* stream, const ConvAOperand* conva, RbKernelLaunch* capture = nullptr);

// rbGemmWorkspaceSize when operand `implicit_operand` (0 = A, 1 = B, -1 = none) is fetched in place by im2col loads
// and therefore needs neither a pitched copy nor TF32 planes inside the GEMM's own workspace.
size_t gemm_workspace_bytes(const RbGemmProblem* p, int implicit_operand);
// TF32 planes of an f32 matrix stack [groups][R][C]: hi (and lo when `split`) with row pitch `pitch` elements;
// with `transpose` the output is [groups][C][pitch >= R]. x = hi + lo, both exactly representable in TF32.
RbStatus f32_planes(const float* src, float* hi, float* lo, int groups, int R, int C, int pitch, bool transpose,
                    bool split, void* stream);

// rbConv / rbConvWorkspaceSize with the result element type overridden (-1: the problem's own). Backward data into a
// dense [pixels][channels] input takes an override (the folded 3-D path asks for an f32 gradient so that the sum over
// its depth taps rounds once), and so does the forward direction with a fused epilogue (`epi`, applied per output
// channel by the GEMM that ends the convolution).
size_t conv_workspace_bytes(const RbConvProblem* p, int result_type);
RbStatus conv_run(const RbConvProblem* p, int result_type, void* filter, void* input, void* output, void* workspace,
                  size_t workspace_bytes, void* stream, const RbEpilogue* epi = nullptr, RbKernelLaunch* capture = nullptr);

// A unit-stride NHWC convolution for conv_halo_run (csrc/conv_halo_sm100.cu): image [N][H][W][C] -> out pixels (n, p, q)
// at element offsets n * o_n + p * o_p + q * o_q with Kout contiguous channels, filter matrix [Kout][(y, x, c)] K-major.
struct HaloConv {
  int N, H, W, C;        // the image tensor that is convolved (input, or the output gradient for backward data)
  int P, Q, Kout;        // output image and channels
  int Y, X, dil_h, dil_w;
  int pad_h, pad_w, pad_h_r, pad_w_r;
  int is_bf16;
  long long o_n, o_p, o_q;
  // Backward data reading the KYXC filter tensor as it lies (no rearranged copy): `filter_matrix` is then the filter
  // itself, [C = conv output channels][FY][FX][Kout = conv input channels, contiguous] with element strides f_sk, f_sy,
  // f_sx, and tap (y', x') of the raster is filter tap (fy0 + fsy * (Y-1-y'), fx0 + fsx * (X-1-x')).
  bool b_mn = false;
  int FY = 0, FX = 0;
  long long f_sk = 0, f_sy = 0, f_sx = 0;
  int fy0 = 0, fsy = 1, fx0 = 0, fsx = 1;
};
bool conv_halo_applicable(const HaloConv& c);
RbStatus conv_halo_run(const HaloConv& c, const void* image, const void* filter_matrix, void* out, void* stream,
                       const RbEpilogue* epi = nullptr, int out_type = -1);
// Up to four such convolutions of the SAME image in one launch (each with its own filter matrix, output pointer and
// pixel strides): the CTAs are divided among them in proportion to their work.
RbStatus conv_halo_run_group(const HaloConv* cs, int count, const void* image, const void* const* filter_matrices,
                             void* const* outs, void* stream, const RbEpilogue* epi = nullptr, int out_type = -1);
// The same forward form with the filter matrix streamed through shared memory (csrc/conv_halo_stream_sm100.cu): any
// channel count; elem_bytes 2 (f16 / bf16, channels-last result) or 4 (f32 as three TF32 products: hi and lo planes of
// the NHWC image and of the K-major filter matrix; the result's channel stride o_k may be 1 or a plane size, NKHW).
bool conv_halo_stream_applicable(const HaloConv& c, int elem_bytes, long long o_k);
RbStatus conv_halo_stream_run(const HaloConv& c, int elem_bytes, const void* image_hi, const void* image_lo, const void* filter_hi,
                              const void* filter_lo, void* out, long long o_k, void* stream);

// Backward weight of the same convolution (csrc/conv_wgrad_halo_sm100.cu): image [N][H][W][C], output gradient
// [N][P][Q][Kout] -> filter gradient [Kout][Y][X][C] in the 16-bit element type. The workspace holds the f32 sums.
// Tuning database (csrc/tuning.cu): the variant word recorded for a problem, 0 = none.
uint32_t tuned_variant_gemm(const RbGemmProblem* p);
uint32_t tuned_variant_conv(const RbConvProblem* p);
// Runs a call under the recorded variant word when the caller set none (nested calls see the outer one).
struct TunedVariantScope {
  int saved;
  bool active;
  explicit TunedVariantScope(uint32_t v) : saved(rbGetGemmVariant()), active(saved == 0 && v != 0) {
    if (active) rbSetGemmVariant((int)v);
  }
  ~TunedVariantScope() {
    if (active) rbSetGemmVariant(saved);
  }
  TunedVariantScope(const TunedVariantScope&) = delete;
  TunedVariantScope& operator=(const TunedVariantScope&) = delete;
};

// GEMM+GEMM with the intermediate kept on the SM (csrc/attention_sm100.cu): k1, n2 <= 128, 16-bit types.
bool gemm_gemm_on_chip_applicable(int32_t k1, int32_t n1, int32_t n2, int32_t data_type);
RbStatus gemm_gemm_on_chip(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type, const void* a,
                           const void* b1, const void* b2, void* o, void* stream);

bool conv_wgrad_halo_applicable(const HaloConv& c);
size_t conv_wgrad_halo_workspace(const HaloConv& c);
RbStatus conv_wgrad_halo_run(const HaloConv& c, const void* image, const void* out_grad, void* filter_grad, void* workspace,
                             size_t workspace_bytes, void* stream);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (device, kernel, size): the call costs microseconds and
// small problems are bound by the host's launch path.
RbStatus ensure_dynamic_smem(const void* kernel, int bytes);

// Device trace buffer set with rbSetTraceBuffer for the calling thread (nullptr when `need` words do not fit).
unsigned long long* trace_buffer(size_t need_u64);

inline size_t dtype_bytes(int t) {
  switch (t) {
    case RB_F32: case RB_I32: return 4;
    case RB_F16: case RB_BF16: return 2;
    case RB_I8: case RB_F8E4M3: case RB_F8E5M2: case RB_F8E4M3_E5M2: case RB_F8E5M2_E4M3: return 1;
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
