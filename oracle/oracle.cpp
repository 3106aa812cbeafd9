// CPU oracle: a restatement of rocMLIR's CPU validation path for the contraction hot path.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product (rocmlir_b200/, the C ABI) may call, link or
// import this file; it is used by tests/, by the smoke check and by the bench's CPU-baseline leg.
//
// The reference's CPU validator is MLIR that rocmlir-gen emits and mlir-cpu-runner JIT-executes
// (mlir/tools/rocmlir-gen/rocmlir-gen.cpp); it cannot be built here without LLVM/MLIR, so each
// function below restates the loop nest, the types and the rounding of the cited generator code.
// Pinning: the convolution functions reproduce the known-answer tensors of
// mlir/test/rocmlir-driver/cpu_conv2d/*.mlir (tests/golden/cpu_conv2d.json), and the verifier and
// RNG functions are compared against the reference's own conv-validation-wrappers.cpp compiled
// into oracle/_ref/ (tests/test_oracle_vs_ref.py).
//
// Build: make -C oracle   (g++ -O2 -ffp-contract=off -fopenmp: no FMA contraction, because the
// generated host code performs mulf and addf as two separately rounded operations).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

// Element types; numbering shared with RbDType in include/rocmlir_b200.h (plus i64 for references).
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_I8 = 3, ORC_I32 = 4, ORC_F8E4M3 = 5, ORC_I64 = 6, ORC_F64 = 7, ORC_F8E5M2 = 8 };

// ------------------------------------------------------------------------------------------------
// Scalar conversions (arith.truncf / arith.extf semantics: round to nearest even)
// ------------------------------------------------------------------------------------------------
static inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

static inline uint16_t f32_to_f16_bits(float f) {
  const uint32_t x = f2u(f);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u) return (uint16_t)(sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to >= 65520 -> inf
  if (ax < 0x33000001u) return (uint16_t)sign;               // <= 2^-25 -> zero (ties to even)
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t he;
  if (e < -14) { shift = 13 + (-14 - e); he = 0; } else { shift = 13; he = (uint32_t)(e + 15); }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  uint32_t h = (he == 0) ? q : ((he << 10) + (q - 0x400u));  // a mantissa carry bumps the exponent
  return (uint16_t)(sign | h);
}
static inline float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return u2f(sign);
    int s = 0;
    while (!(m & 0x400u)) { m <<= 1; s++; }
    m &= 0x3FFu;
    return u2f(sign | ((uint32_t)(127 - 15 - s + 1) << 23) | (m << 13));
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
static inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t x = f2u(f);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7FFFu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}
static inline float bf16_bits_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

// OCP e4m3fn: bias 7, no inf, NaN = S.1111.111, max finite 448. f32 -> e4m3 is round-to-nearest-even
// followed by saturation to +-448 (mlir/lib/Conversion/EmulateFp8ExtTrunc/EmulateFp8ExtTrunc.cpp:208-218
// with saturateFP8Truncf = true, mlir/lib/Dialect/Rock/Pipelines/Pipelines.cpp:238); NaN stays NaN.
static inline float e4m3_bits_to_f32(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
  float r;
  if (e == 15 && m == 7) r = std::numeric_limits<float>::quiet_NaN();
  else if (e == 0) r = std::ldexp((float)m, -9);
  else r = std::ldexp((float)(8 + m), e - 10);
  return s ? -r : r;
}
static inline uint8_t f32_to_e4m3_bits(float f) {
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  if (std::isnan(f)) return sign | 0x7F;
  const float a = std::fabs(f);
  if (a >= 448.0f) return sign | 0x7E;  // includes inf and everything that would round above 448 (464 tie -> sat)
  if (a < std::ldexp(1.0f, -10)) return sign;          // below half of the smallest subnormal (2^-9) -> 0 (tie to even)
  int e;
  std::frexp(a, &e);        // a = frac * 2^e, frac in [0.5,1)
  int ue = e - 1;           // unbiased exponent of the leading bit
  if (ue < -6) ue = -6;     // subnormal range shares the scale 2^-6 * 2^-3
  const float scaled = std::ldexp(a, 3 - ue);  // in units of the last mantissa bit
  float q = std::nearbyint(scaled);            // default rounding mode: ties to even
  int qi = (int)q;
  int be = ue + 7;
  if (ue == -6 && qi < 8) return sign | (uint8_t)qi;  // subnormal
  if (qi == 16) { qi = 8; be += 1; }
  if (be > 15 || (be == 15 && qi - 8 == 7)) return sign | 0x7E;
  return sign | (uint8_t)((be << 3) | (qi - 8));
}

// OCP e5m2: the upper byte of an IEEE half (bias 15, inf and NaN exist, max finite 57344). f32 -> e5m2 is
// round-to-nearest-even on the 2-bit mantissa, then saturation to +-57344 like the e4m3 truncation above.
static inline float e5m2_bits_to_f32(uint8_t v) { return f16_bits_to_f32((uint16_t)((uint16_t)v << 8)); }
static inline uint8_t f32_to_e5m2_bits(float f) {
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  if (std::isnan(f)) return sign | 0x7F;
  const float a = std::fabs(f);
  if (a >= 57344.0f) return sign | 0x7B;        // max finite (everything at or above it, inf included, saturates)
  if (a < std::ldexp(1.0f, -17)) return sign;   // below half of the smallest subnormal (2^-16)
  int e;
  std::frexp(a, &e);
  int ue = e - 1;
  if (ue < -14) ue = -14;                       // subnormals share the scale 2^-14 * 2^-2
  const float scaled = std::ldexp(a, 2 - ue);   // in units of the last mantissa bit
  int qi = (int)std::nearbyint(scaled);         // ties to even
  int be = ue + 15;
  if (ue == -14 && qi < 4) return sign | (uint8_t)qi;
  if (qi == 8) { qi = 4; be += 1; }
  if (be >= 31) return sign | 0x7B;
  return sign | (uint8_t)((be << 2) | (qi - 4));
}

static inline float round_to(float x, int t) {
  switch (t) {
    case ORC_F16: return f16_bits_to_f32(f32_to_f16_bits(x));
    case ORC_BF16: return bf16_bits_to_f32(f32_to_bf16_bits(x));
    case ORC_F8E4M3: return e4m3_bits_to_f32(f32_to_e4m3_bits(x));
    case ORC_F8E5M2: return e5m2_bits_to_f32(f32_to_e5m2_bits(x));
    default: return x;
  }
}

ORC_API void orc_convert_to_f32(const void* src, int dtype, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    switch (dtype) {
      case ORC_F32: dst[i] = ((const float*)src)[i]; break;
      case ORC_F16: dst[i] = f16_bits_to_f32(((const uint16_t*)src)[i]); break;
      case ORC_BF16: dst[i] = bf16_bits_to_f32(((const uint16_t*)src)[i]); break;
      case ORC_I8: dst[i] = (float)((const int8_t*)src)[i]; break;
      case ORC_I32: dst[i] = (float)((const int32_t*)src)[i]; break;
      case ORC_F8E4M3: dst[i] = e4m3_bits_to_f32(((const uint8_t*)src)[i]); break;
      case ORC_F8E5M2: dst[i] = e5m2_bits_to_f32(((const uint8_t*)src)[i]); break;
      case ORC_I64: dst[i] = (float)((const int64_t*)src)[i]; break;
      default: dst[i] = 0; break;
    }
  }
}

// float -> integer as tosa.cast lowers it: round half to even, then clamp to the destination range
// (external/llvm-project/mlir/lib/Conversion/TosaToLinalg/TosaToLinalg.cpp:497-555). NaN -> 0.
static inline int64_t f32_to_int_sat(float x, int64_t lo, int64_t hi) {
  if (std::isnan(x)) return 0;
  const float r = std::nearbyint(x);
  if (r <= (float)lo) return lo;
  if (r >= (float)hi) return hi;
  return (int64_t)r;
}

// rocmlir-gen stores random / pattern values with arith.fptosi (ints) or arith.truncf (small floats)
// (rocmlir-gen.cpp:1474-1480). `sat_int` selects the tosa.cast rule instead of plain fptosi.
ORC_API void orc_convert_from_f32(const float* src, void* dst, int dtype, int64_t n, int sat_int) {
  for (int64_t i = 0; i < n; ++i) {
    const float x = src[i];
    switch (dtype) {
      case ORC_F32: ((float*)dst)[i] = x; break;
      case ORC_F16: ((uint16_t*)dst)[i] = f32_to_f16_bits(x); break;
      case ORC_BF16: ((uint16_t*)dst)[i] = f32_to_bf16_bits(x); break;
      case ORC_I8: ((int8_t*)dst)[i] = sat_int ? (int8_t)f32_to_int_sat(x, -128, 127) : (int8_t)(int32_t)x; break;
      case ORC_I32: ((int32_t*)dst)[i] = sat_int ? (int32_t)f32_to_int_sat(x, INT32_MIN, INT32_MAX) : (int32_t)x; break;
      case ORC_F8E4M3: ((uint8_t*)dst)[i] = f32_to_e4m3_bits(x); break;
      case ORC_F8E5M2: ((uint8_t*)dst)[i] = f32_to_e5m2_bits(x); break;
      default: break;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Data fill (conv-validation-wrappers.cpp:27-50; rocmlir-gen.cpp:1325-1486, 3157-3218)
// ------------------------------------------------------------------------------------------------
ORC_API void orc_seed(uint32_t seed) {
  if (seed == 0) std::srand((unsigned)time(0));
  else std::srand(seed);
}
ORC_API float orc_random_integer_value(int16_t mn, int16_t mx) {
  if (mn == mx) return mn;
  int16_t v = (int16_t)((std::rand() % (mx - mn)) + mn);
  return (float)v;
}
ORC_API float orc_random_float_value(int16_t mn, int16_t mx) {
  const float minf = (float)mn;
  if (mn == mx) return (float)(minf * 0.1);
  return (float)((mx - mn) * (double)std::rand() / (double)RAND_MAX) + minf;
}
// One libc rand() per element, tensors filled in kernel-argument order, each flattened row-major.
ORC_API void orc_fill_random(float* dst, int64_t n, int rand_float, int16_t mn, int16_t mx) {
  for (int64_t i = 0; i < n; ++i) dst[i] = rand_float ? orc_random_float_value(mn, mx) : orc_random_integer_value(mn, mx);
}
// -rand fixed / none: pattern cycled over the flat index (rocmlir-gen.cpp:1359-1425).
ORC_API void orc_fill_pattern(float* dst, int64_t n, const float* pattern, int plen) {
  for (int64_t i = 0; i < n; ++i) dst[i] = pattern[i % plen];
}

// ------------------------------------------------------------------------------------------------
// GEMM (rocmlir-gen.cpp:2401-2493): loops g, m, n, k (k innermost, ascending); float: f32 multiply
// then f32 add; integer: operands sign-extended to i64, exact. Inputs are the f32-widened copies the
// generator makes; truncation to C's element type happens on copy-out (orc_convert_from_f32).
// ------------------------------------------------------------------------------------------------
ORC_API void orc_gemm_f32(const float* a, const float* b, float* c, int64_t G, int64_t M, int64_t N, int64_t K, int ta,
                          int tb, int tc, int threads) {
#pragma omp parallel for collapse(2) num_threads(threads > 0 ? threads : 1) schedule(static)
  for (int64_t g = 0; g < G; ++g)
    for (int64_t m = 0; m < M; ++m) {
      const float* ag = a + g * M * K;
      const float* bg = b + g * K * N;
      float* cg = c + g * M * N;
      for (int64_t n = 0; n < N; ++n) {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; ++k) {
          const float av = ta ? ag[k * M + m] : ag[m * K + k];
          const float bv = tb ? bg[n * K + k] : bg[k * N + n];
          const float mul = av * bv;
          acc = acc + mul;
        }
        cg[tc ? n * M + m : m * N + n] = acc;
      }
    }
}
ORC_API void orc_gemm_i8(const int8_t* a, const int8_t* b, int64_t* c, int64_t G, int64_t M, int64_t N, int64_t K,
                         int ta, int tb, int tc, int threads) {
#pragma omp parallel for collapse(2) num_threads(threads > 0 ? threads : 1) schedule(static)
  for (int64_t g = 0; g < G; ++g)
    for (int64_t m = 0; m < M; ++m) {
      const int8_t* ag = a + g * M * K;
      const int8_t* bg = b + g * K * N;
      int64_t* cg = c + g * M * N;
      for (int64_t n = 0; n < N; ++n) {
        int64_t acc = 0;
        for (int64_t k = 0; k < K; ++k) {
          const int64_t av = ta ? ag[k * M + m] : ag[m * K + k];
          const int64_t bv = tb ? bg[n * K + k] : bg[k * N + n];
          acc += av * bv;
        }
        cg[tc ? n * M + m : m * N + n] = acc;
      }
    }
}
// Reference in double precision, used only to report error against an accuracy oracle.
ORC_API void orc_gemm_f64(const float* a, const float* b, double* c, int64_t G, int64_t M, int64_t N, int64_t K, int ta,
                          int tb, int tc, int threads) {
#pragma omp parallel for collapse(2) num_threads(threads > 0 ? threads : 1) schedule(static)
  for (int64_t g = 0; g < G; ++g)
    for (int64_t m = 0; m < M; ++m) {
      const float* ag = a + g * M * K;
      const float* bg = b + g * K * N;
      double* cg = c + g * M * N;
      for (int64_t n = 0; n < N; ++n) {
        double acc = 0.0;
        for (int64_t k = 0; k < K; ++k)
          acc += (double)(ta ? ag[k * M + m] : ag[m * K + k]) * (double)(tb ? bg[n * K + k] : bg[k * N + n]);
        cg[tc ? n * M + m : m * N + n] = acc;
      }
    }
}

// ------------------------------------------------------------------------------------------------
// Convolution (rocmlir-gen.cpp:1715-1997). Canonical 5-D tensors with a group dimension, each in any
// memory permutation, given here by element strides for the named dimensions:
//   filter (g,k,c,y,x)   input (n,g,c,h,w)   output (n,g,k,ho,wo)
// The loop nest runs over the RESULT tensor's dimensions, then the reduction channel, then the
// reduction image dimensions, so each result element accumulates in a fixed order:
//   fwd:        c, y, x        in_h = ho*stride_h + y*dil_h - pad_h   (skip when outside the image)
//   bwd-weight: n, ho, wo      same index relation
//   bwd-data:   k, y, x        t = in_h + pad_h - y*dil_h; needs t % stride_h == 0, ho = t/stride_h in range
// f32 multiply then f32 add. The result is zero-filled first.
// ------------------------------------------------------------------------------------------------
struct OrcConv {
  int64_t n, g, c, k, h, w, y, x, ho, wo;
  int64_t stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;  // pad_* are the left paddings
  int64_t fs[5], is[5], os[5];
};

template <typename TIn, typename TAcc, bool kWrapI8>
static void conv_impl(const OrcConv& p, int dir, const TIn* fil, const TIn* in, const TIn* out, TAcc* res, int threads) {
  auto F = [&](int64_t g, int64_t k, int64_t c, int64_t y, int64_t x) {
    return g * p.fs[0] + k * p.fs[1] + c * p.fs[2] + y * p.fs[3] + x * p.fs[4];
  };
  auto I = [&](int64_t n, int64_t g, int64_t c, int64_t h, int64_t w) {
    return n * p.is[0] + g * p.is[1] + c * p.is[2] + h * p.is[3] + w * p.is[4];
  };
  auto O = [&](int64_t n, int64_t g, int64_t k, int64_t h, int64_t w) {
    return n * p.os[0] + g * p.os[1] + k * p.os[2] + h * p.os[3] + w * p.os[4];
  };
  auto mac = [](TAcc acc, TIn a, TIn b) -> TAcc {
    if constexpr (std::is_floating_point<TAcc>::value) {
      const TAcc mul = (TAcc)a * (TAcc)b;
      return acc + mul;
    } else if constexpr (kWrapI8) {
      // The generated reference multiplies the two i8 values in i8 and only then sign-extends
      // (arith.muli on i8, arith.extsi; rocmlir-gen.cpp:1955-1960): the product wraps modulo 256.
      const int8_t mul = (int8_t)((int)a * (int)b);
      return acc + (TAcc)mul;
    } else {
      return acc + (TAcc)a * (TAcc)b;
    }
  };
  const int nt = threads > 0 ? threads : 1;
  if (dir == 0) {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t n = 0; n < p.n; ++n)
      for (int64_t g = 0; g < p.g; ++g)
        for (int64_t k = 0; k < p.k; ++k)
          for (int64_t ho = 0; ho < p.ho; ++ho)
            for (int64_t wo = 0; wo < p.wo; ++wo) {
              TAcc acc = 0;
              for (int64_t c = 0; c < p.c; ++c)
                for (int64_t y = 0; y < p.y; ++y)
                  for (int64_t x = 0; x < p.x; ++x) {
                    const int64_t ih = ho * p.stride_h + y * p.dil_h - p.pad_h;
                    const int64_t iw = wo * p.stride_w + x * p.dil_w - p.pad_w;
                    if (ih < 0 || ih >= p.h || iw < 0 || iw >= p.w) continue;
                    acc = mac(acc, fil[F(g, k, c, y, x)], in[I(n, g, c, ih, iw)]);
                  }
              res[O(n, g, k, ho, wo)] = acc;
            }
  } else if (dir == 2) {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t g = 0; g < p.g; ++g)
      for (int64_t k = 0; k < p.k; ++k)
        for (int64_t c = 0; c < p.c; ++c)
          for (int64_t y = 0; y < p.y; ++y)
            for (int64_t x = 0; x < p.x; ++x) {
              TAcc acc = 0;
              for (int64_t n = 0; n < p.n; ++n)
                for (int64_t ho = 0; ho < p.ho; ++ho)
                  for (int64_t wo = 0; wo < p.wo; ++wo) {
                    const int64_t ih = ho * p.stride_h + y * p.dil_h - p.pad_h;
                    const int64_t iw = wo * p.stride_w + x * p.dil_w - p.pad_w;
                    if (ih < 0 || ih >= p.h || iw < 0 || iw >= p.w) continue;
                    acc = mac(acc, out[O(n, g, k, ho, wo)], in[I(n, g, c, ih, iw)]);
                  }
              res[F(g, k, c, y, x)] = acc;
            }
  } else {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t n = 0; n < p.n; ++n)
      for (int64_t g = 0; g < p.g; ++g)
        for (int64_t c = 0; c < p.c; ++c)
          for (int64_t ih = 0; ih < p.h; ++ih)
            for (int64_t iw = 0; iw < p.w; ++iw) {
              TAcc acc = 0;
              for (int64_t k = 0; k < p.k; ++k)
                for (int64_t y = 0; y < p.y; ++y)
                  for (int64_t x = 0; x < p.x; ++x) {
                    const int64_t th = ih + p.pad_h - y * p.dil_h;
                    const int64_t tw = iw + p.pad_w - x * p.dil_w;
                    if (th < 0 || tw < 0 || th % p.stride_h || tw % p.stride_w) continue;
                    const int64_t ho = th / p.stride_h, wo = tw / p.stride_w;
                    if (ho >= p.ho || wo >= p.wo) continue;
                    acc = mac(acc, fil[F(g, k, c, y, x)], out[O(n, g, k, ho, wo)]);
                  }
              res[I(n, g, c, ih, iw)] = acc;
            }
  }
}

// dir: 0 fwd (res = output), 1 bwd-data (res = input), 2 bwd-weight (res = filter).
ORC_API void orc_conv_f32(const OrcConv* p, int dir, const float* fil, const float* in, const float* out, float* res,
                          int threads) {
  conv_impl<float, float, false>(*p, dir, fil, in, out, res, threads);
}
// i8 forward only (rocmlir-gen.cpp:2019-2024), i64 result. wrap_product = 1 is the reference's behaviour.
ORC_API void orc_conv_i8(const OrcConv* p, const int8_t* fil, const int8_t* in, int64_t* res, int wrap_product,
                         int threads) {
  if (wrap_product) conv_impl<int8_t, int64_t, true>(*p, 0, fil, in, nullptr, res, threads);
  else conv_impl<int8_t, int64_t, false>(*p, 0, fil, in, nullptr, res, threads);
}
ORC_API void orc_conv_f64(const OrcConv* p, int dir, const float* fil, const float* in, const float* out, double* res,
                          int threads) {
  conv_impl<float, double, false>(*p, dir, fil, in, out, res, threads);
}

// ------------------------------------------------------------------------------------------------
// Convolution with three image dimensions: the same generated loop nest with nImageDims = 3
// (rocmlir-gen.cpp:1745-1830). Image dimensions are numbered 0 = h, 1 = w, 2 = d
// (parseConvTensorLayout, rocmlir-gen.cpp:1504-1542), and the reduction loops run in that order after the
// reduction channel, so the depth tap is the innermost loop:
//   fwd: c, y, x, z      bwd-weight: n, ho, wo, do      bwd-data: k, y, x, z
// Strides for filter (g,k,c,z,y,x), input (n,g,c,d,h,w), output (n,g,k,do,ho,wo).
// ------------------------------------------------------------------------------------------------
struct OrcConv3 {
  int64_t n, g, c, k, d, h, w, z, y, x, dout, ho, wo;
  int64_t stride_d, stride_h, stride_w, dil_d, dil_h, dil_w, pad_d, pad_h, pad_w;  // left paddings
  int64_t fs[6], is[6], os[6];
};

template <typename TIn, typename TAcc>
static void conv3_impl(const OrcConv3& p, int dir, const TIn* fil, const TIn* in, const TIn* out, TAcc* res, int threads) {
  auto F = [&](int64_t g, int64_t k, int64_t c, int64_t z, int64_t y, int64_t x) {
    return g * p.fs[0] + k * p.fs[1] + c * p.fs[2] + z * p.fs[3] + y * p.fs[4] + x * p.fs[5];
  };
  auto I = [&](int64_t n, int64_t g, int64_t c, int64_t d, int64_t h, int64_t w) {
    return n * p.is[0] + g * p.is[1] + c * p.is[2] + d * p.is[3] + h * p.is[4] + w * p.is[5];
  };
  auto O = [&](int64_t n, int64_t g, int64_t k, int64_t d, int64_t h, int64_t w) {
    return n * p.os[0] + g * p.os[1] + k * p.os[2] + d * p.os[3] + h * p.os[4] + w * p.os[5];
  };
  auto mac = [](TAcc acc, TIn a, TIn b) -> TAcc {
    const TAcc mul = (TAcc)a * (TAcc)b;
    return acc + mul;
  };
  const int nt = threads > 0 ? threads : 1;
  if (dir == 0) {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t n = 0; n < p.n; ++n)
      for (int64_t g = 0; g < p.g; ++g)
        for (int64_t k = 0; k < p.k; ++k)
          for (int64_t od = 0; od < p.dout; ++od)
            for (int64_t ho = 0; ho < p.ho; ++ho)
              for (int64_t wo = 0; wo < p.wo; ++wo) {
                TAcc acc = 0;
                for (int64_t c = 0; c < p.c; ++c)
                  for (int64_t y = 0; y < p.y; ++y)
                    for (int64_t x = 0; x < p.x; ++x)
                      for (int64_t z = 0; z < p.z; ++z) {
                        const int64_t ih = ho * p.stride_h + y * p.dil_h - p.pad_h;
                        const int64_t iw = wo * p.stride_w + x * p.dil_w - p.pad_w;
                        const int64_t id = od * p.stride_d + z * p.dil_d - p.pad_d;
                        if (ih < 0 || ih >= p.h || iw < 0 || iw >= p.w || id < 0 || id >= p.d) continue;
                        acc = mac(acc, fil[F(g, k, c, z, y, x)], in[I(n, g, c, id, ih, iw)]);
                      }
                res[O(n, g, k, od, ho, wo)] = acc;
              }
  } else if (dir == 2) {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t g = 0; g < p.g; ++g)
      for (int64_t k = 0; k < p.k; ++k)
        for (int64_t c = 0; c < p.c; ++c)
          for (int64_t z = 0; z < p.z; ++z)
            for (int64_t y = 0; y < p.y; ++y)
              for (int64_t x = 0; x < p.x; ++x) {
                TAcc acc = 0;
                for (int64_t n = 0; n < p.n; ++n)
                  for (int64_t ho = 0; ho < p.ho; ++ho)
                    for (int64_t wo = 0; wo < p.wo; ++wo)
                      for (int64_t od = 0; od < p.dout; ++od) {
                        const int64_t ih = ho * p.stride_h + y * p.dil_h - p.pad_h;
                        const int64_t iw = wo * p.stride_w + x * p.dil_w - p.pad_w;
                        const int64_t id = od * p.stride_d + z * p.dil_d - p.pad_d;
                        if (ih < 0 || ih >= p.h || iw < 0 || iw >= p.w || id < 0 || id >= p.d) continue;
                        acc = mac(acc, out[O(n, g, k, od, ho, wo)], in[I(n, g, c, id, ih, iw)]);
                      }
                res[F(g, k, c, z, y, x)] = acc;
              }
  } else {
#pragma omp parallel for collapse(3) num_threads(nt) schedule(static)
    for (int64_t n = 0; n < p.n; ++n)
      for (int64_t g = 0; g < p.g; ++g)
        for (int64_t c = 0; c < p.c; ++c)
          for (int64_t id = 0; id < p.d; ++id)
            for (int64_t ih = 0; ih < p.h; ++ih)
              for (int64_t iw = 0; iw < p.w; ++iw) {
                TAcc acc = 0;
                for (int64_t k = 0; k < p.k; ++k)
                  for (int64_t y = 0; y < p.y; ++y)
                    for (int64_t x = 0; x < p.x; ++x)
                      for (int64_t z = 0; z < p.z; ++z) {
                        const int64_t th = ih + p.pad_h - y * p.dil_h;
                        const int64_t tw = iw + p.pad_w - x * p.dil_w;
                        const int64_t td = id + p.pad_d - z * p.dil_d;
                        if (th < 0 || tw < 0 || td < 0 || th % p.stride_h || tw % p.stride_w || td % p.stride_d) continue;
                        const int64_t ho = th / p.stride_h, wo = tw / p.stride_w, od = td / p.stride_d;
                        if (ho >= p.ho || wo >= p.wo || od >= p.dout) continue;
                        acc = mac(acc, fil[F(g, k, c, z, y, x)], out[O(n, g, k, od, ho, wo)]);
                      }
                res[I(n, g, c, id, ih, iw)] = acc;
              }
  }
}

ORC_API void orc_conv3d_f32(const OrcConv3* p, int dir, const float* fil, const float* in, const float* out, float* res,
                            int threads) {
  conv3_impl<float, float>(*p, dir, fil, in, out, res, threads);
}
ORC_API void orc_conv3d_f64(const OrcConv3* p, int dir, const float* fil, const float* in, const float* out, double* res,
                            int threads) {
  conv3_impl<float, double>(*p, dir, fil, in, out, res, threads);
}
// i8 forward with the operands widened before the product (exact integer arithmetic)
ORC_API void orc_conv3d_i8(const OrcConv3* p, const int8_t* fil, const int8_t* in, int64_t* res, int threads) {
  conv3_impl<int8_t, int64_t>(*p, 0, fil, in, nullptr, res, threads);
}

// ------------------------------------------------------------------------------------------------
// Attention (rocmlir-gen.cpp:2507-2638; op order pinned by mlir/test/rocmlir-gen/attention-kernel.mlir).
// Every TOSA op is typed with the element type T, and tosa.matmul accumulates in its RESULT type
// (external/llvm-project/mlir/lib/Conversion/TosaToLinalg/TosaToLinalgNamed.cpp:645-657), so with
// T = f16 every multiply, add, exp and reciprocal is rounded to f16. Inputs here are f32 arrays that
// already hold T-representable values:
//   Q [G,Sq,D], K [G,D,Sk], V [G,Sk,Dv], optional scale/bias [G,Sq,Sk], optional mask (i8, [G,Sq,Sk],
//   `where(mask != 0, S, fill)` as MIGraphX expresses masking), O [G,Sq,Dv].
//   S = matmul(Q,K); S *= scale; S += bias; S = where(mask); m = max_k S; E = exp(S - m);
//   l = sum_k E; P = E * reciprocal(l); O = matmul(P, V)
// elem_type ORC_F32 / ORC_F16 / ORC_BF16 selects T; ORC_F64 evaluates everything in double.
// A scalar `scale_scalar` (used when scale == NULL and use_scalar != 0) is the MIGraphX literal form.
// ------------------------------------------------------------------------------------------------
ORC_API void orc_attention(const float* q, const float* k, const float* v, const float* scale, const float* bias,
                           const int8_t* mask, float mask_fill, int use_scalar, float scale_scalar, float* o,
                           int64_t G, int64_t Sq, int64_t Sk, int64_t D, int64_t Dv, int elem_type, int causal,
                           int64_t g_begin, int64_t g_end, int threads) {
  const int nt = threads > 0 ? threads : 1;
  const bool f64 = elem_type == ORC_F64;
#pragma omp parallel for collapse(2) num_threads(nt) schedule(static)
  for (int64_t g = g_begin; g < g_end; ++g)
    for (int64_t i = 0; i < Sq; ++i) {
      std::vector<double> sd(f64 ? Sk : 0);
      std::vector<float> s(f64 ? 0 : Sk);
      const float* qg = q + (g * Sq + i) * D;
      const float* kg = k + g * D * Sk;
      const float* vg = v + g * Sk * Dv;
      float* og = o + (g * Sq + i) * Dv;
      if (f64) {
        double mx = -INFINITY;
        for (int64_t j = 0; j < Sk; ++j) {
          double acc = 0;
          for (int64_t d = 0; d < D; ++d) acc += (double)qg[d] * (double)kg[d * Sk + j];
          if (scale) acc *= scale[(g * Sq + i) * Sk + j];
          else if (use_scalar) acc *= (double)scale_scalar;
          if (bias) acc += bias[(g * Sq + i) * Sk + j];
          if (mask && mask[(g * Sq + i) * Sk + j] == 0) acc = mask_fill;
          if (causal && j > i) acc = -INFINITY;
          sd[j] = acc;
          mx = std::max(mx, acc);
        }
        double l = 0;
        for (int64_t j = 0; j < Sk; ++j) { sd[j] = std::exp(sd[j] - mx); l += sd[j]; }
        for (int64_t d = 0; d < Dv; ++d) {
          double acc = 0;
          for (int64_t j = 0; j < Sk; ++j) acc += sd[j] / l * (double)vg[j * Dv + d];
          og[d] = (float)acc;
        }
        continue;
      }
      const int T = elem_type;
      float mx = -INFINITY;
      for (int64_t j = 0; j < Sk; ++j) {
        float acc = 0.0f;
        for (int64_t d = 0; d < D; ++d) {
          const float mul = round_to(qg[d] * kg[d * Sk + j], T);
          acc = round_to(acc + mul, T);
        }
        if (scale) acc = round_to(acc * scale[(g * Sq + i) * Sk + j], T);
        else if (use_scalar) acc = round_to(acc * scale_scalar, T);
        if (bias) acc = round_to(acc + bias[(g * Sq + i) * Sk + j], T);
        if (mask && mask[(g * Sq + i) * Sk + j] == 0) acc = mask_fill;
        if (causal && j > i) acc = -INFINITY;
        s[j] = acc;
        mx = std::max(mx, acc);
      }
      float l = 0.0f;
      for (int64_t j = 0; j < Sk; ++j) {
        const float e = round_to(std::exp(round_to(s[j] - mx, T)), T);
        s[j] = e;
        l = round_to(l + e, T);
      }
      const float rl = round_to(1.0f / l, T);
      for (int64_t j = 0; j < Sk; ++j) s[j] = round_to(s[j] * rl, T);
      for (int64_t d = 0; d < Dv; ++d) {
        float acc = 0.0f;
        for (int64_t j = 0; j < Sk; ++j) {
          const float mul = round_to(s[j] * vg[j * Dv + d], T);
          acc = round_to(acc + mul, T);
        }
        og[d] = acc;
      }
    }
}

// First-GEMM-quantised attention (rocmlir-gen -t i8: Q and K are i8, everything else f16; generator
// rocmlir-gen.cpp:3497-3515, CPU reference :2562-2581): tosa.matmul i8 x i8 -> i32, minus the i8 quantisation bias
// widened to i32, cast to f16, times the f16 quantisation scale; from there on the f16 chain of orc_attention.
// quant_bias and quant_scale are the single elements of their 1x1x1 tensors.
ORC_API void orc_attention_i8(const int8_t* q, const int8_t* k, const float* v, int quant_bias, float quant_scale,
                              const float* scale, const float* bias, float* o, int64_t G, int64_t Sq, int64_t Sk,
                              int64_t D, int64_t Dv, int threads) {
  const int nt = threads > 0 ? threads : 1;
  const int T = ORC_F16;
#pragma omp parallel for collapse(2) num_threads(nt) schedule(static)
  for (int64_t g = 0; g < G; ++g)
    for (int64_t i = 0; i < Sq; ++i) {
      std::vector<float> s(Sk);
      const int8_t* qg = q + (g * Sq + i) * D;
      const int8_t* kg = k + g * D * Sk;
      const float* vg = v + g * Sk * Dv;
      float* og = o + (g * Sq + i) * Dv;
      float mx = -INFINITY;
      for (int64_t j = 0; j < Sk; ++j) {
        int32_t acc_i = 0;
        for (int64_t d = 0; d < D; ++d) acc_i += (int32_t)qg[d] * (int32_t)kg[d * Sk + j];
        acc_i -= (int32_t)quant_bias;
        float acc = round_to((float)acc_i, T);
        acc = round_to(acc * quant_scale, T);
        if (scale) acc = round_to(acc * scale[(g * Sq + i) * Sk + j], T);
        if (bias) acc = round_to(acc + bias[(g * Sq + i) * Sk + j], T);
        s[j] = acc;
        mx = std::max(mx, acc);
      }
      float l = 0.0f;
      for (int64_t j = 0; j < Sk; ++j) {
        const float e = round_to(std::exp(round_to(s[j] - mx, T)), T);
        s[j] = e;
        l = round_to(l + e, T);
      }
      const float rl = round_to(1.0f / l, T);
      for (int64_t j = 0; j < Sk; ++j) s[j] = round_to(s[j] * rl, T);
      for (int64_t d = 0; d < Dv; ++d) {
        float acc = 0.0f;
        for (int64_t j = 0; j < Sk; ++j) {
          const float mul = round_to(s[j] * vg[j * Dv + d], T);
          acc = round_to(acc + mul, T);
        }
        og[d] = acc;
      }
    }
}

// gemm + gemm: O = (A.B1).B2 with the intermediate rounded to the element type, the behaviour of
// the attention skeleton with softmax removed
// (mlir/lib/Dialect/Rock/Transforms/GridwiseGemmToBlockwise.cpp:1790-1813, 2162-2165). f32 accumulation
// for both products (accumulator rule of GemmToGridwise.cpp:93-109), k ascending.
ORC_API void orc_gemm_gemm(const float* a, const float* b1, const float* b2, float* o, int64_t M, int64_t K1,
                           int64_t N1, int64_t N2, int mid_type, int threads) {
  const int nt = threads > 0 ? threads : 1;
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    std::vector<float> t(N1);
    for (int64_t n = 0; n < N1; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K1; ++k) { const float mul = a[m * K1 + k] * b1[k * N1 + n]; acc = acc + mul; }
      t[n] = round_to(acc, mid_type);
    }
    for (int64_t n = 0; n < N2; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < N1; ++k) { const float mul = t[k] * b2[k * N2 + n]; acc = acc + mul; }
      o[m * N2 + n] = acc;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Fused elementwise tail, op by op (MIGraphXToTosa.cpp:876-1018; tosa.cast rule above):
//   x = acc (f32; integer accumulators converted with sitofp = RNE)
//   [round to mid_type]  [x *= alpha]  [x *= col_scale[n]]  [x += bias[n]; round to mid_type]
//   [x = max(x,0)]  [x *= out_recip]   -> f32 result; the caller converts to the stored type with
//   orc_convert_from_f32(..., sat_int = 1).
// flags use the RB_EPI_* bit values of include/rocmlir_b200.h.
// ------------------------------------------------------------------------------------------------
ORC_API void orc_epilogue(const float* acc_f32, const int64_t* acc_i64, float* out, int64_t rows, int64_t N,
                          uint32_t flags, float alpha, const float* col_scale, const float* bias, float out_recip,
                          int mid_type, float clip_lo, float clip_hi, float in_zero, const float* residual, int unary) {
  // flags: 1 alpha, 2 col_scale, 4 bias (256: indexed by the row, 512: a scalar), 8 relu, 16 requant, 32 round to
  // mid_type, 64 clip (tosa.maximum then tosa.minimum, MIGraphXToTosa.cpp:1089-1101), 128 same-shape add,
  // 1024 dequantisation zero point: (cast(x) - cast(zp)) * scale (MIGraphXToTosa.cpp:879-902),
  // 4096 one unary elementwise function (MIGraphX.td:134-181; 1 abs 2 ceil 3 erf 4 exp 5 floor 6 log 7 neg 8 recip 9 rsqrt
  // 10 sigmoid = 1 / (1 + exp(-x)) 11 sqrt 12 tanh) evaluated in f32 with the C library, result rounded to mid_type
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t n = 0; n < N; ++n) {
      float x = acc_i64 ? (float)(int32_t)acc_i64[r * N + n] : acc_f32[r * N + n];
      if (flags & 1024) x = x - in_zero;
      if (flags & 32) x = round_to(x, mid_type);
      if (flags & 1) x = x * alpha;
      if (flags & 2) x = x * col_scale[n];
      if (flags & 4) {
        x = x + bias[(flags & 512) ? 0 : (flags & 256) ? r : n];
        if (flags & 32) x = round_to(x, mid_type);
      }
      if (flags & 128) { x = x + residual[r * N + n]; if (flags & 32) x = round_to(x, mid_type); }
      if (flags & 4096) {
        switch (unary) {
          case 1: x = std::fabs(x); break;
          case 2: x = std::ceil(x); break;
          case 3: x = std::erf(x); break;
          case 4: x = std::exp(x); break;
          case 5: x = std::floor(x); break;
          case 6: x = std::log(x); break;
          case 7: x = -x; break;
          case 8: x = 1.0f / x; break;
          case 9: x = 1.0f / std::sqrt(x); break;
          case 10: x = 1.0f / (1.0f + std::exp(-x)); break;
          case 11: x = std::sqrt(x); break;
          case 12: x = std::tanh(x); break;
          default: break;
        }
        if (flags & 32) x = round_to(x, mid_type);
      }
      if (flags & 8) x = x > 0.0f ? x : 0.0f;
      if (flags & 64) { x = x > clip_lo ? x : clip_lo; x = x < clip_hi ? x : clip_hi; }
      if (flags & 16) x = x * out_recip;
      out[r * N + n] = x;
    }
}

// ------------------------------------------------------------------------------------------------
// Verification (conv-validation-wrappers.cpp:104-216 for floats, :232-285 for integers).
// metrics[0] = RMS, [1] = max abs diff, [2] = max rel diff. Returns bit0 RMS ok, bit1 abs ok, bit2 rel ok.
// ------------------------------------------------------------------------------------------------
ORC_API int orc_verify_float(const float* gpu, const float* val, int64_t n, float thr_rms, float thr_abs,
                             float thr_rel, double* metrics) {
  float max_abs = 0.0f, max_mag = 0.0f;
  double max_rel = 0.0, sum_sq = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    float v = val[i];
    const float g = gpu[i];
    max_mag = std::max(max_mag, std::max(std::fabs(v), std::fabs(g)));
    if (v == g) continue;
    if (std::isinf(v)) v = v > 0 ? 65504.0f : -65504.0f;
    const float d = std::fabs(v - g);
    if (d > max_abs) max_abs = d;
    if (v != 0.0f) {
      const double rel = (double)d / (double)std::fabs(v);
      if (rel > max_rel) max_rel = rel;
    }
    sum_sq += (double)d * (double)d;
  }
  const double rms = std::sqrt(sum_sq) / ((double)max_mag * std::sqrt((double)n));
  if (metrics) { metrics[0] = rms; metrics[1] = max_abs; metrics[2] = max_rel; }
  return (rms <= thr_rms ? 1 : 0) | (max_abs <= thr_abs ? 2 : 0) | (max_rel <= thr_rel ? 4 : 0);
}
// Exact equality; counts[0] = mismatches, counts[1] = reference values that do not fit the tested type.
ORC_API int orc_verify_int(const void* gpu, int gpu_type, const int64_t* val, int64_t n, int64_t* counts) {
  int64_t fail = 0, ovf = 0;
  const int64_t lo = gpu_type == ORC_I8 ? -128 : INT32_MIN, hi = gpu_type == ORC_I8 ? 127 : INT32_MAX;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t g = gpu_type == ORC_I8 ? (int64_t)((const int8_t*)gpu)[i] : (int64_t)((const int32_t*)gpu)[i];
    if (val[i] > hi || val[i] < lo) ovf++;
    if (g != val[i]) fail++;
  }
  if (counts) { counts[0] = fail; counts[1] = ovf; }
  return fail == 0 ? 7 : 0;
}

ORC_API int orc_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
