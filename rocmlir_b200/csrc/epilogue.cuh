// Fused elementwise epilogue evaluated on accumulator values held in registers (TMEM -> registers ->
// HBM). The step order and the per-step rounding are part of the library's contract (see RbEpilogue in
// include/rocmlir_b200.h); they restate what rocMLIR's fused linalg.generic readers compute
// (mlir/lib/Dialect/Rock/Transforms/AlignTiling.cpp:903-1049 with the MIGraphX lowerings in
// mlir/lib/Conversion/MIGraphXToTosa/MIGraphXToTosa.cpp:876-1018).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/rocmlir_b200.h"

namespace rb {

struct EpiParams {
  uint32_t flags;
  float alpha;
  float out_recip;
  int mid_type;
  int bias_type;
  const float* col_scale;
  const void* bias;
};

__device__ __forceinline__ float round_to_type(float x, int t) {
  if (t == RB_F16) return __half2float(__float2half_rn(x));
  if (t == RB_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

__device__ __forceinline__ float load_bias(const void* bias, int bias_type, long long n) {
  if (bias_type == RB_F16) return __half2float(reinterpret_cast<const __half*>(bias)[n]);
  if (bias_type == RB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
  return reinterpret_cast<const float*>(bias)[n];
}

// One accumulator element -> epilogue value (still f32). `n` is the global column (bias / scale index).
// No FMA contraction: every multiply and add is its own correctly rounded f32 operation.
__device__ __forceinline__ float epi_apply(float x, const EpiParams& e, long long n) {
  if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  if (e.flags & RB_EPI_ALPHA) x = __fmul_rn(x, e.alpha);
  if (e.flags & RB_EPI_COL_SCALE) x = __fmul_rn(x, __ldg(e.col_scale + n));
  if (e.flags & RB_EPI_BIAS) {
    x = __fadd_rn(x, load_bias(e.bias, e.bias_type, n));
    if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  }
  if (e.flags & RB_EPI_RELU) x = fmaxf(x, 0.0f);
  if (e.flags & RB_EPI_REQUANT) x = __fmul_rn(x, e.out_recip);
  return x;
}

// The same steps on 32 consecutive columns held in registers, one uniform branch per step instead of per element.
// `cs` / `bs` point at the 32 per-column scales / biases of these columns, already converted to f32 (shared memory).
__device__ __forceinline__ void epi_apply32(float* x, const EpiParams& e, const float* cs, const float* bs) {
  if (e.flags & RB_EPI_ROUND_MID) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = round_to_type(x[j], e.mid_type);
  }
  if (e.flags & RB_EPI_ALPHA) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = __fmul_rn(x[j], e.alpha);
  }
  if (e.flags & RB_EPI_COL_SCALE) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 s4 = *reinterpret_cast<const float4*>(cs + j);
      x[j] = __fmul_rn(x[j], s4.x); x[j + 1] = __fmul_rn(x[j + 1], s4.y);
      x[j + 2] = __fmul_rn(x[j + 2], s4.z); x[j + 3] = __fmul_rn(x[j + 3], s4.w);
    }
  }
  if (e.flags & RB_EPI_BIAS) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b4 = *reinterpret_cast<const float4*>(bs + j);
      x[j] = __fadd_rn(x[j], b4.x); x[j + 1] = __fadd_rn(x[j + 1], b4.y);
      x[j + 2] = __fadd_rn(x[j + 2], b4.z); x[j + 3] = __fadd_rn(x[j + 3], b4.w);
    }
    if (e.flags & RB_EPI_ROUND_MID) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = round_to_type(x[j], e.mid_type);
    }
  }
  if (e.flags & RB_EPI_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
  }
  if (e.flags & RB_EPI_REQUANT) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = __fmul_rn(x[j], e.out_recip);
  }
}

// float -> integer cast of tosa.cast: round half to even, then saturate
// (external/llvm-project/mlir/lib/Conversion/TosaToLinalg/TosaToLinalg.cpp:497-555).
__device__ __forceinline__ int f32_to_int_sat(float x, int lo, int hi) {
  int v = __float2int_rn(x);  // saturates at the i32 range, NaN -> 0
  return min(max(v, lo), hi);
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ int dtype_size(int t) {
  return (t == RB_F32 || t == RB_I32) ? 4 : ((t == RB_F16 || t == RB_BF16) ? 2 : 1);
}

// Store one f32 value to element index `idx` of a buffer of type `t`.
__device__ __forceinline__ void store_elem(void* base, long long idx, float x, int t) {
  switch (t) {
    case RB_F32: reinterpret_cast<float*>(base)[idx] = x; break;
    case RB_F16: reinterpret_cast<__half*>(base)[idx] = __float2half_rn(x); break;
    case RB_BF16: reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x); break;
    case RB_I8: reinterpret_cast<int8_t*>(base)[idx] = static_cast<int8_t>(f32_to_int_sat(x, -128, 127)); break;
    case RB_I32: reinterpret_cast<int32_t*>(base)[idx] = f32_to_int_sat(x, INT32_MIN, INT32_MAX); break;
    case RB_F8E4M3: reinterpret_cast<uint8_t*>(base)[idx] = f32_to_e4m3(x); break;
    default: break;
  }
}

// Packs 32 consecutive f32 values into the C type: 8 (4-byte types), 4 (2-byte) or 2 (1-byte) 16-byte
// words in `out`; returns that count.
__device__ __forceinline__ int pack_row32(const float* x, int t, uint4* out) {
  if (t == RB_F32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = make_uint4(__float_as_uint(x[4 * i]), __float_as_uint(x[4 * i + 1]), __float_as_uint(x[4 * i + 2]),
                          __float_as_uint(x[4 * i + 3]));
    return 8;
  }
  if (t == RB_I32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = make_uint4((uint32_t)f32_to_int_sat(x[4 * i], INT32_MIN, INT32_MAX),
                          (uint32_t)f32_to_int_sat(x[4 * i + 1], INT32_MIN, INT32_MAX),
                          (uint32_t)f32_to_int_sat(x[4 * i + 2], INT32_MIN, INT32_MAX),
                          (uint32_t)f32_to_int_sat(x[4 * i + 3], INT32_MIN, INT32_MAX));
    return 8;
  }
  if (t == RB_F16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 h = __floats2half2_rn(x[8 * i + 2 * j], x[8 * i + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      out[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return 4;
  }
  if (t == RB_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x[8 * i + 2 * j], x[8 * i + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      out[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return 4;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {  // 8-bit outputs
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t b = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v = x[16 * i + 4 * j + k];
        const uint32_t byte =
            (t == RB_I8) ? (uint32_t)(uint8_t)(int8_t)f32_to_int_sat(v, -128, 127) : (uint32_t)f32_to_e4m3(v);
        b |= byte << (8 * k);
      }
      w[j] = b;
    }
    out[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return 2;
}

}  // namespace rb
