// int4 weights: migraphx.unpack (+ dequantizelinear) in front of a contraction.
//
// rocMLIR carries packed 4-bit operands up to the kernel boundary (mlir/include/mlir/Dialect/MIGraphX/IR/MIGraphX.td:183-212,
// mlir/lib/Dialect/MIGraphX/Transforms/RealizeInt4.cpp) and fuses the unpack and the dequantisation into the
// contraction's operand loads. Here the same two steps run as one pass that writes the operand in its element type
// into the caller's workspace, and the contraction reads that:
//     out[2 i]     = (lo(in[i]) - zero) * scale
//     out[2 i + 1] = (hi(in[i]) - zero) * scale        lo = in & 0xf, hi = in >> 4 (arithmetic shift when signed)
// rounded once to the output type (the int4 value and the difference are exact, so one rounding of the product is what
// an f16 / bf16 / f32 multiply gives). out_type RB_I8: the plain unpack (scale and zero point are not applied).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "lib_state.h"

namespace rb {
namespace {

template <typename T>
__device__ __forceinline__ T cvt_out(float x);
template <>
__device__ __forceinline__ __half cvt_out<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ float cvt_out<float>(float x) { return x; }

__device__ __forceinline__ void nibbles(uint8_t b, bool is_unsigned, int& lo, int& hi) {
  if (is_unsigned) {
    lo = b & 0xf;
    hi = b >> 4;
  } else {
    lo = (int)((int8_t)(b << 4)) >> 4;   // sign-extend the low nibble
    hi = (int)((int8_t)b) >> 4;
  }
}

template <typename T>
__global__ void unpack_int4_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, long long nbytes, int is_unsigned,
                                   float scale, int zero) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nbytes; i += (long long)gridDim.x * blockDim.x) {
    int lo, hi;
    nibbles(in[i], is_unsigned != 0, lo, hi);
    out[2 * i] = cvt_out<T>(__fmul_rn((float)(lo - zero), scale));
    out[2 * i + 1] = cvt_out<T>(__fmul_rn((float)(hi - zero), scale));
  }
}

__global__ void unpack_int4_i8_kernel(const uint8_t* __restrict__ in, int8_t* __restrict__ out, long long nbytes, int is_unsigned) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nbytes; i += (long long)gridDim.x * blockDim.x) {
    int lo, hi;
    nibbles(in[i], is_unsigned != 0, lo, hi);
    out[2 * i] = (int8_t)lo;
    out[2 * i + 1] = (int8_t)hi;
  }
}

}  // namespace
}  // namespace rb

extern "C" RbStatus rbUnpackInt4(const void* packed, void* out, int64_t packed_bytes, int32_t is_unsigned, int32_t out_type,
                                 float scale, int32_t zero_point, void* stream_v) {
  using namespace rb;
  if (!packed || !out) return fail(RB_INVALID_PARAM, "packed and out must be device pointers");
  if (packed_bytes < 0) return fail(RB_INVALID_PARAM, "negative size");
  if (packed_bytes == 0) return RB_SUCCESS;
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int blocks = (int)std::min<long long>((packed_bytes + 255) / 256, (long long)dev->sm_count * 16);
  const uint8_t* in = static_cast<const uint8_t*>(packed);
  switch (out_type) {
    case RB_I8: unpack_int4_i8_kernel<<<blocks, 256, 0, stream>>>(in, static_cast<int8_t*>(out), packed_bytes, is_unsigned); break;
    case RB_F16: unpack_int4_kernel<__half><<<blocks, 256, 0, stream>>>(in, static_cast<__half*>(out), packed_bytes, is_unsigned, scale, zero_point); break;
    case RB_BF16: unpack_int4_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(in, static_cast<__nv_bfloat16*>(out), packed_bytes, is_unsigned, scale, zero_point); break;
    case RB_F32: unpack_int4_kernel<float><<<blocks, 256, 0, stream>>>(in, static_cast<float*>(out), packed_bytes, is_unsigned, scale, zero_point); break;
    default: return fail(RB_UNSUPPORTED, "int4 operands are unpacked to i8, f16, bf16 or f32");
  }
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  return RB_SUCCESS;
}
