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
  float clip_lo, clip_hi;   // RB_EPI_CLIP
  float in_zero;            // RB_EPI_ZP_IN: zero point of the dequantisation, already cast to f32
  int out_zero;             // RB_EPI_ZP_OUT: zero point added after the rounding cast of the quantisation
  const void* residual;     // RB_EPI_RESIDUAL: tensor of C's shape and layout, element type res_type
  int res_type;
  int unary;                // RB_EPI_UNARY: RbUnary
};

// A bias vector indexed by the output column (the per-column vectors are staged in shared memory by the GEMM kernel).
__host__ __device__ __forceinline__ bool epi_col_bias(uint32_t flags) {
  return (flags & RB_EPI_BIAS) && !(flags & (RB_EPI_BIAS_ROW | RB_EPI_BIAS_SCALAR));
}
__host__ __device__ __forceinline__ bool epi_needs_col_vectors(uint32_t flags) {
  return (flags & RB_EPI_COL_SCALE) || epi_col_bias(flags);
}

__device__ __forceinline__ float round_to_type(float x, int t) {
  if (t == RB_F16) return __half2float(__float2half_rn(x));
  if (t == RB_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

// The MIGraphX unary elementwise ops in f32 (MIGraphX.td:134-181). sigmoid = 1 / (1 + exp(-x)) as
// MIGraphXToTosa lowers it; recip and rsqrt are correctly rounded divisions / square roots, not the approximate forms.
__device__ __forceinline__ float epi_unary(float x, int op) {
  switch (op) {
    case RB_UNARY_ABS: return fabsf(x);
    case RB_UNARY_CEIL: return ceilf(x);
    case RB_UNARY_ERF: return erff(x);
    case RB_UNARY_EXP: return expf(x);
    case RB_UNARY_FLOOR: return floorf(x);
    case RB_UNARY_LOG: return logf(x);
    case RB_UNARY_NEG: return -x;
    case RB_UNARY_RECIP: return __fdiv_rn(1.0f, x);
    case RB_UNARY_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case RB_UNARY_SIGMOID: return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
    case RB_UNARY_SQRT: return __fsqrt_rn(x);
    case RB_UNARY_TANH: return tanhf(x);
    default: return x;
  }
}

__device__ __forceinline__ float load_bias(const void* bias, int bias_type, long long n) {
  if (bias_type == RB_F16) return __half2float(reinterpret_cast<const __half*>(bias)[n]);
  if (bias_type == RB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n]);
  return reinterpret_cast<const float*>(bias)[n];
}

// One accumulator element -> epilogue value (still f32). `n` / `m` are the global column and row (bias / scale
// indices), `idx` the element's index in C's layout (residual index).
// No FMA contraction: every multiply and add is its own correctly rounded f32 operation.
__device__ __forceinline__ float epi_apply(float x, const EpiParams& e, long long n, long long m, long long idx) {
  if (e.flags & RB_EPI_ZP_IN) x = __fsub_rn(x, e.in_zero);
  if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  if (e.flags & RB_EPI_ALPHA) x = __fmul_rn(x, e.alpha);
  if (e.flags & RB_EPI_COL_SCALE) x = __fmul_rn(x, __ldg(e.col_scale + n));
  if (e.flags & RB_EPI_BIAS) {
    const long long bi = (e.flags & RB_EPI_BIAS_SCALAR) ? 0 : (e.flags & RB_EPI_BIAS_ROW) ? m : n;
    x = __fadd_rn(x, load_bias(e.bias, e.bias_type, bi));
    if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  }
  if (e.flags & RB_EPI_RESIDUAL) {
    x = __fadd_rn(x, load_bias(e.residual, e.res_type, idx));
    if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  }
  if (e.flags & RB_EPI_UNARY) {
    x = epi_unary(x, e.unary);
    if (e.flags & RB_EPI_ROUND_MID) x = round_to_type(x, e.mid_type);
  }
  if (e.flags & RB_EPI_RELU) x = fmaxf(x, 0.0f);
  if (e.flags & RB_EPI_CLIP) x = fminf(fmaxf(x, e.clip_lo), e.clip_hi);
  if (e.flags & RB_EPI_REQUANT) x = __fmul_rn(x, e.out_recip);
  return x;
}

// What the thread that owns one row of a tile knows besides the per-column vectors: its row's bias (row / scalar
// bias modes) and where the residual elements of its 32 columns lie.
struct EpiRow {
  float row_bias = 0.0f;
  const void* res = nullptr;   // residual element of (row, first column); nullptr: row outside the matrix
  long long res_stride = 1;    // elements between consecutive columns
  int ncols = 32;              // columns of the 32 that exist
};

// The same steps on 32 consecutive columns held in registers, one uniform branch per step instead of per element.
// `cs` / `bs` point at the 32 per-column scales / biases of these columns, already converted to f32 (shared memory).
__device__ __forceinline__ void epi_apply32(float* x, const EpiParams& e, const float* cs, const float* bs,
                                            const EpiRow& r) {
  if (e.flags & RB_EPI_ZP_IN) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = __fsub_rn(x[j], e.in_zero);
  }
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
    if (e.flags & (RB_EPI_BIAS_ROW | RB_EPI_BIAS_SCALAR)) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = __fadd_rn(x[j], r.row_bias);
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 b4 = *reinterpret_cast<const float4*>(bs + j);
        x[j] = __fadd_rn(x[j], b4.x); x[j + 1] = __fadd_rn(x[j + 1], b4.y);
        x[j + 2] = __fadd_rn(x[j + 2], b4.z); x[j + 3] = __fadd_rn(x[j + 3], b4.w);
      }
    }
    if (e.flags & RB_EPI_ROUND_MID) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = round_to_type(x[j], e.mid_type);
    }
  }
  if (e.flags & RB_EPI_RESIDUAL) {
    if (r.res) {
      const int es = (e.res_type == RB_F32) ? 4 : 2;
      const bool vec = r.res_stride == 1 && r.ncols == 32 && (reinterpret_cast<uintptr_t>(r.res) & 15) == 0;
      if (vec && es == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 w = __ldg(reinterpret_cast<const uint4*>(r.res) + i);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float lo, hi;
            if (e.res_type == RB_F16) {
              const __half2 h = *reinterpret_cast<const __half2*>(&ww[j]);
              lo = __low2float(h); hi = __high2float(h);
            } else {
              const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&ww[j]);
              lo = __low2float(h); hi = __high2float(h);
            }
            x[8 * i + 2 * j] = __fadd_rn(x[8 * i + 2 * j], lo);
            x[8 * i + 2 * j + 1] = __fadd_rn(x[8 * i + 2 * j + 1], hi);
          }
        }
      } else if (vec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(r.res) + i);
          x[4 * i] = __fadd_rn(x[4 * i], w.x); x[4 * i + 1] = __fadd_rn(x[4 * i + 1], w.y);
          x[4 * i + 2] = __fadd_rn(x[4 * i + 2], w.z); x[4 * i + 3] = __fadd_rn(x[4 * i + 3], w.w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < r.ncols) x[j] = __fadd_rn(x[j], load_bias(r.res, e.res_type, (long long)j * r.res_stride));
      }
    }
    if (e.flags & RB_EPI_ROUND_MID) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = round_to_type(x[j], e.mid_type);
    }
  }
  if (e.flags & RB_EPI_UNARY) {
#pragma unroll 4
    for (int j = 0; j < 32; ++j) x[j] = epi_unary(x[j], e.unary);
    if (e.flags & RB_EPI_ROUND_MID) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = round_to_type(x[j], e.mid_type);
    }
  }
  if (e.flags & RB_EPI_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
  }
  if (e.flags & RB_EPI_CLIP) {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = fminf(fmaxf(x[j], e.clip_lo), e.clip_hi);
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
// quantizelinear with a zero point (MIGraphXToTosa.cpp:923-978): cast to i32 (round half even, saturating), add the
// zero point as an i32 add, clamp to the i8 range.
__device__ __forceinline__ int f32_to_i8_zp(float x, int zp) {
  const int v = (int)((unsigned)__float2int_rn(x) + (unsigned)zp);
  return min(max(v, -128), 127);
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ int dtype_size(int t) {
  return (t == RB_F32 || t == RB_I32) ? 4 : ((t == RB_F16 || t == RB_BF16) ? 2 : 1);
}

// Store one f32 value to element index `idx` of a buffer of type `t`.
__device__ __forceinline__ void store_elem(void* base, long long idx, float x, int t, int zp = 0) {
  switch (t) {
    case RB_F32: reinterpret_cast<float*>(base)[idx] = x; break;
    case RB_F16: reinterpret_cast<__half*>(base)[idx] = __float2half_rn(x); break;
    case RB_BF16: reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x); break;
    case RB_I8: reinterpret_cast<int8_t*>(base)[idx] = static_cast<int8_t>(f32_to_i8_zp(x, zp)); break;
    case RB_I32: reinterpret_cast<int32_t*>(base)[idx] = f32_to_int_sat(x, INT32_MIN, INT32_MAX); break;
    case RB_F8E4M3: reinterpret_cast<uint8_t*>(base)[idx] = f32_to_e4m3(x); break;
    default: break;
  }
}

// Packs 32 consecutive f32 values into the C type: 8 (4-byte types), 4 (2-byte) or 2 (1-byte) 16-byte
// words in `out`; returns that count.
__device__ __forceinline__ int pack_row32(const float* x, int t, uint4* out, int zp = 0) {
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
            (t == RB_I8) ? (uint32_t)(uint8_t)(int8_t)f32_to_i8_zp(v, zp) : (uint32_t)f32_to_e4m3(v);
        b |= byte << (8 * k);
      }
      w[j] = b;
    }
    out[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return 2;
}

}  // namespace rb
