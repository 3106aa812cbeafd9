// rock.attention on sm_100a: O = softmax(f(Q.K)) . V per group, flash style (one pass over the keys with a
// running row maximum and row sum), both matrix products on tcgen05 with accumulators in TMEM.
//
// Replaces what rocMLIR generates for rock.attention (GridwiseAttentionAccelRewritePattern,
// mlir/lib/Dialect/Rock/Transforms/GridwiseGemmToBlockwise.cpp:743-2403): one workgroup per slab of queries, a
// loop over key blocks, S = Q.K on the matrix unit, the pre-softmax elementwise region f (scale, bias, mask)
// applied to the score tile in registers, exp2 with the log2(e) factor folded into the scale (:2085-2093),
// running max / sum (:1087-1148), O rescaled when the maximum moves (:1207-1261), O / sum at the end
// (:2338-2356). Differences by design: the row statistics are f32 (the reference keeps them in the element
// type), and a causal mask can be given analytically instead of as a [G,Sq,Sk] tensor.
//
// Element types: f16 and bf16 on the kernels below; the first-GEMM-quantised form of rocmlir-gen -t i8 on the same
// kernels after widening Q and K to f16 (exact), with the reference's f16 rounding chain reproduced in f; f32 on a
// separate unfused true-f32 path (attention_f32). Operands stored transposed (transQ / transV / transO) and K rows
// off 16-byte boundaries are re-strided in scratch first.
//
// CTA = one 128-row query tile, 256 threads:
//   warp 0   producer: TMA loads of Q (once) and of the K and V tiles of each key block (2-deep rings)
//   warp 1   MMA issuer: S_j = Q.K_j^T into one of two TMEM score buffers, O += P_j.V_j
//   warp 2   TMEM allocator
//   warps 4-7 softmax: thread = query row (TMEM lane). The 128 scores of the row are read from TMEM once, P = exp2(x - m)
//            is written back over the score buffer in the element type (two values per 32-bit column) and is the
//            A operand of P.V straight from TMEM; O is rescaled in TMEM only when the running maximum has grown by
//            more than 2^8 since the reference maximum was last moved (exp2 stays in range, the final O / l
//            cancels the stale reference); final O / l and TMA store.
// S_{j+1} is issued before P_j is awaited, so the score MMA of the next block overlaps the softmax of this one.
// MMAs of one issuing thread execute in order, which is what makes P_j safe in the buffer S_{j+2} will overwrite.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "epilogue.cuh"
#include "lib_state.h"
#include "ptx.cuh"

namespace rb {
namespace {

constexpr int kQT = 128;    // query rows per CTA
constexpr int kKT = 128;    // keys per block
constexpr int kAttThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct AttMaps {
  CUtensorMap q, k, v, o;
};

struct AttParams {
  int G, Sq, Sk, D, Dv;
  int trans_k;       // K stored [G][Sk][D] (K-major) instead of [G][D][Sk]
  int is_bf16;
  int causal;
  int q_tiles;
  float scale_log2;  // scale * log2(e)
  const void* bias;  // optional additive [G][Sq][Sk], element type
  const void* scale_t;  // optional multiplicative [G][Sq][Sk], element type (applied before the bias)
  const int8_t* mask;  // optional [G][Sq][Sk]: score kept where mask != 0, else mask_fill
  float mask_fill;
  uint32_t idesc_s, idesc_pv;
  uint32_t* status;
  const void* quant_bias;      // first-GEMM-quantised form: device pointers to one i8 and one f16 (else null)
  const void* quant_scale;
  unsigned long long* trace;   // optional [CTAs][16] cycle counters (two-tile kernel), see rbSetTraceBuffer
  int linear;        // GEMM+GEMM: P = S rounded to the element type (no scale, no softmax, no division by a row sum)
};

struct AttSmem {
  static constexpr int kQBytes = kQT * 256;        // up to D = 128 f16
  static constexpr int kKBytes = kKT * 256;
  static constexpr int kVBytes = kKT * 256;
  static constexpr int kStages = 3;
  static constexpr int kQ = 0;                     // reused as the store staging area at the end
  static constexpr int kK = kQ + kQBytes;
  static constexpr int kV = kK + kStages * kKBytes;
  static constexpr int kBars = kV + kStages * kVBytes;
  static constexpr int kTotal = kBars + 256 + 1024;
};

__device__ __forceinline__ float load_elem(const void* p, long long i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                 : __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float f16_round(float x) { return __half2float(__float2half_rn(x)); }

__global__ void __launch_bounds__(kAttThreads, 1) attention_fwd_kernel(const __grid_constant__ AttMaps maps,
                                                                        const AttParams p) {
  constexpr int NS = AttSmem::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::kBars);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;             // [NS]
  uint64_t* k_empty = k_full + NS;         // [NS]
  uint64_t* v_full = k_empty + NS;         // [NS]
  uint64_t* v_empty = v_full + NS;         // [NS]
  uint64_t* s_full = v_empty + NS;         // [2]
  uint64_t* p_full = s_full + 2;
  uint64_t* pv_done = p_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = lane_id();
  const int g = blockIdx.x / p.q_tiles;
  // long tiles first under a causal mask
  const int qt = p.causal ? (p.q_tiles - 1 - blockIdx.x % p.q_tiles) : (blockIdx.x % p.q_tiles);
  const int q0 = qt * kQT;
  int nb = (p.Sk + kKT - 1) / kKT;
  if (p.causal) nb = min(nb, (min(q0 + kQT, p.Sq) - 1) / kKT + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<1>(tmem_holder, 512);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&maps.q);
    prefetch_tmap(&maps.k);
    prefetch_tmap(&maps.v);
    prefetch_tmap(&maps.o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_o = tmem_base + 256;   // S buffers at columns 0 and 128, O at 256

  const int d_atoms = p.D / 64, dv_chunks = p.Dv / 64;
  const uint32_t q_bytes = (uint32_t)kQT * p.D * 2, k_bytes = (uint32_t)kKT * p.D * 2, v_bytes = (uint32_t)kKT * p.Dv * 2;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, q_bytes);
      for (int a = 0; a < d_atoms; ++a) tma_load_3d(smem + AttSmem::kQ + a * (kQT * 128), &maps.q, q_full, a * 64, q0, g);
      int s = 0;
      uint32_t par = 0;
      for (int j = 0; j < nb; ++j) {
        if (!mbar_wait(&k_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + s)) break;
        uint8_t* ks = smem + AttSmem::kK + s * AttSmem::kKBytes;
        mbar_expect_tx(&k_full[s], k_bytes);
        if (p.trans_k) {
          for (int a = 0; a < d_atoms; ++a) tma_load_3d(ks + a * (kKT * 128), &maps.k, &k_full[s], a * 64, j * kKT, g);
        } else {
          for (int c = 0; c < kKT / 64; ++c) tma_load_3d(ks + c * (p.D * 128), &maps.k, &k_full[s], j * kKT + c * 64, 0, g);
        }
        if (!mbar_wait(&v_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + 4 + s)) break;
        uint8_t* vs = smem + AttSmem::kV + s * AttSmem::kVBytes;
        mbar_expect_tx(&v_full[s], v_bytes);
        for (int c = 0; c < dv_chunks; ++c) tma_load_3d(vs + c * (kKT * 128), &maps.v, &v_full[s], c * 64, j * kKT, g);
        if (++s == NS) { s = 0; par ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_addr = smem_u32(smem + AttSmem::kQ);
      int ks_stage = 0;        // ring position of the next K tile to consume
      uint32_t ks_par = 0;
      auto issue_s = [&](int j) -> bool {
        if (!mbar_wait(&k_full[ks_stage], ks_par, p.status, kStatusTimeoutMma + ks_stage)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + AttSmem::kK + ks_stage * AttSmem::kKBytes);
        const int ksteps = p.D / 16;
        for (int kk = 0; kk < ksteps; ++kk) {
          const uint32_t a_lo = smem_desc_lo(q_addr + (kk >> 2) * (kQT * 128) + (kk & 3) * 32, 16);
          const uint32_t b_lo = p.trans_k ? smem_desc_lo(k_addr + (kk >> 2) * (kKT * 128) + (kk & 3) * 32, 16)
                                          : smem_desc_lo(k_addr + kk * 2048, (uint32_t)p.D * 128);
          umma_ss<kKindF16, 1>(tmem_base + (j & 1) * 128, desc64(a_lo, hi), desc64(b_lo, hi), p.idesc_s, kk ? 1u : 0u);
        }
        tc_commit<1>(&s_full[j & 1]);
        tc_commit<1>(&k_empty[ks_stage]);
        if (++ks_stage == NS) { ks_stage = 0; ks_par ^= 1u; }
        return true;
      };
      bool ok = mbar_wait(q_full, 0, p.status, kStatusTimeoutMma + 8);
      if (ok) ok = issue_s(0);
      int vs_stage = 0;
      uint32_t vs_par = 0;
      for (int j = 0; j < nb && ok; ++j) {
        // S_{j+1} goes into the buffer that held S_{j-1} / P_{j-1}; P_{j-1}.V_{j-1} was issued before it and MMAs
        // execute in issue order.
        if (j + 1 < nb) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(p_full, (uint32_t)j & 1u, p.status, kStatusTimeoutMma + 9)) break;
        if (!mbar_wait(&v_full[vs_stage], vs_par, p.status, kStatusTimeoutMma + 10 + vs_stage)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + AttSmem::kV + vs_stage * AttSmem::kVBytes);
        const uint32_t tmem_p = tmem_base + (j & 1) * 128;   // P_j: 128 lanes x 64 columns, two values per column
        for (int kk = 0; kk < kKT / 16; ++kk) {
          const uint32_t b_lo = smem_desc_lo(v_addr + kk * 2048, kKT * 128);
          umma_ts<kKindF16>(tmem_o, tmem_p + kk * 8, desc64(b_lo, hi), p.idesc_pv, (j | kk) ? 1u : 0u);
        }
        tc_commit<1>(pv_done);
        tc_commit<1>(&v_empty[vs_stage]);
        if (++vs_stage == NS) { vs_stage = 0; vs_par ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int wq = warp & 3;
    const int r = wq * 32 + lane;          // row within the tile == TMEM lane
    const long long row = (long long)q0 + r;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    float m_ref = -INFINITY;   // maximum the exponentials are taken against
    const float qbias = p.quant_bias ? (float)*static_cast<const int8_t*>(p.quant_bias) : 0.0f;
    const float qscale = p.quant_scale ? __half2float(*static_cast<const __half*>(p.quant_scale)) : 1.0f;
    float l = 0.0f;
    bool ok = true;
    for (int j = 0; j < nb && ok; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(&s_full[sb], (uint32_t)(j >> 1) & 1u, p.status, kStatusTimeoutEpilogue + sb)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_s = tmem_base + lane_base + sb * 128;
      const int key0 = j * kKT;
      const bool side_inputs = p.bias || p.mask || p.scale_t || p.quant_scale;          // per-element tensors: general path
      const bool edge = (key0 + kKT > p.Sk) || (p.causal && key0 + kKT - 1 > q0);  // key tail or diagonal block
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + c * 32, v + c * 32);
      tmem_ld_wait();
      if (p.linear) {
        // GEMM+GEMM: the intermediate is S itself in the element type; columns past the end of N1 are zero
        const int limit = p.Sk - key0;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          v[i] = pack2((2 * i < limit) ? __uint_as_float(v[2 * i]) : 0.0f, (2 * i + 1 < limit) ? __uint_as_float(v[2 * i + 1]) : 0.0f, p.is_bf16);
        tmem_st32(tmem_s, v);
        tmem_st32(tmem_s + 32, v + 32);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        l = 1.0f;
        continue;
      }
      // f(S) in the log2 domain: scale, bias, masks
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      if (!side_inputs && !edge) {
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          const float x0 = __uint_as_float(v[i]) * p.scale_log2, x1 = __uint_as_float(v[i + 1]) * p.scale_log2;
          const float x2 = __uint_as_float(v[i + 2]) * p.scale_log2, x3 = __uint_as_float(v[i + 3]) * p.scale_log2;
          v[i] = __float_as_uint(x0); v[i + 1] = __float_as_uint(x1); v[i + 2] = __float_as_uint(x2); v[i + 3] = __float_as_uint(x3);
          mx0 = fmaxf(mx0, x0); mx1 = fmaxf(mx1, x1); mx2 = fmaxf(mx2, x2); mx3 = fmaxf(mx3, x3);
        }
      } else if (!side_inputs) {
        // keys past the end of the sequence or above the diagonal are dropped with a select
        const int limit = min(p.Sk - key0, p.causal ? (int)min(row - key0 + 1, (long long)kKT) : kKT);
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          const float x0 = (i < limit) ? __uint_as_float(v[i]) * p.scale_log2 : -INFINITY;
          const float x1 = (i + 1 < limit) ? __uint_as_float(v[i + 1]) * p.scale_log2 : -INFINITY;
          const float x2 = (i + 2 < limit) ? __uint_as_float(v[i + 2]) * p.scale_log2 : -INFINITY;
          const float x3 = (i + 3 < limit) ? __uint_as_float(v[i + 3]) * p.scale_log2 : -INFINITY;
          v[i] = __float_as_uint(x0); v[i + 1] = __float_as_uint(x1); v[i + 2] = __float_as_uint(x2); v[i + 3] = __float_as_uint(x3);
          mx0 = fmaxf(mx0, x0); mx1 = fmaxf(mx1, x1); mx2 = fmaxf(mx2, x2); mx3 = fmaxf(mx3, x3);
        }
      } else {
        const long long side_off = ((long long)g * p.Sq + min(row, (long long)p.Sq - 1)) * p.Sk;
#pragma unroll
        for (int i = 0; i < 128; ++i) {  // fully unrolled: v[] must stay in registers
          float x = __uint_as_float(v[i]);
          const int key = key0 + i;
          if (p.quant_scale && key < p.Sk) {
            // quantised form: every rounding of the reference's f16 chain is reproduced (see the two-tile kernel)
            x = f16_round(f16_round(x - qbias) * qscale);
            if (p.scale_t) x = f16_round(x * load_elem(p.scale_t, side_off + key, 0));
            if (p.bias) x = f16_round(x + load_elem(p.bias, side_off + key, 0));
            if (p.mask && p.mask[side_off + key] == 0) x = p.mask_fill;
            x *= p.scale_log2;
          } else if (key < p.Sk) {
            x *= p.scale_log2;
            if (p.scale_t) x *= load_elem(p.scale_t, side_off + key, p.is_bf16);
            if (p.bias) x = fmaf(load_elem(p.bias, side_off + key, p.is_bf16), kLog2e, x);
            if (p.mask && p.mask[side_off + key] == 0) x = p.mask_fill * kLog2e;
            if (p.causal && key > row) x = -INFINITY;
          } else {
            x = -INFINITY;
          }
          v[i] = __float_as_uint(x);
          mx0 = fmaxf(mx0, x);
        }
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // Move the reference maximum only when it is first set or the row maximum has outgrown it by more than 2^8.
      float alpha = 1.0f;
      if (mx > m_ref + 8.0f || (m_ref == -INFINITY && mx > -INFINITY)) {
        alpha = ex2(m_ref - mx);   // 0 when the reference was -inf
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;   // a row masked so far keeps exp2 finite (p = 0)
      float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const float p0 = ex2(__uint_as_float(v[2 * i]) - m_use), p1 = ex2(__uint_as_float(v[2 * i + 1]) - m_use);
        const float p2 = ex2(__uint_as_float(v[2 * i + 2]) - m_use), p3 = ex2(__uint_as_float(v[2 * i + 3]) - m_use);
        l0 += p0; l1 += p1; l2 += p2; l3 += p3;
        v[i] = pack2(p0, p1, p.is_bf16);
        v[i + 1] = pack2(p2, p3, p.is_bf16);
      }
      l = l * alpha + ((l0 + l1) + (l2 + l3));
      // P_j over the first 64 columns of the score buffer
      tmem_st32(tmem_s, v);
      tmem_st32(tmem_s + 32, v + 32);
      // rescale O where a reference maximum moved (whole warp takes part: TMEM access is warp-collective)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        if (!mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, p.status, kStatusTimeoutEpilogue + 4)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < p.Dv / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_base + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_o + lane_base + c * 32, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> element type -> staging (the Q tile is no longer needed) -> TMA store ----
    if (ok && mbar_wait(pv_done, (uint32_t)(nb - 1) & 1u, p.status, kStatusTimeoutEpilogue + 5)) {
      tc_fence_after();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      uint8_t* stg = smem + AttSmem::kQ + wq * (2 * 32 * 128);   // per warp: Dv/64 tiles of 32 rows x 128 bytes
#pragma unroll 1
      for (int c = 0; c < p.Dv / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_base + c * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, p.is_bf16);
        uint8_t* rowp = stg + (c >> 1) * (32 * 128) + lane * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int piece = (c & 1) * 4 + i;
          *reinterpret_cast<uint4*>(rowp + ((piece ^ (lane & 7)) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0 && q0 + wq * 32 < p.Sq) {
        for (int c = 0; c < p.Dv / 64; ++c) tma_store_3d(&maps.o, stg + c * (32 * 128), c * 64, q0 + wq * 32, g);
        bulk_commit();
        bulk_wait<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA. One softmax group alone leaves the tensor pipe idle while it works: P_j.V_j has to wait
// for softmax(j). With two 128-row query tiles (A, B) that share every K/V tile, the products of one tile run while
// the other tile's softmax group computes:   ... PV_A(j)  S_A(j+1)  PV_B(j)  S_B(j+1) ...
// 384 threads: warp 0 producer, warp 1 MMA issuer, warp 2 TMEM allocator, warps 4-7 softmax of tile A, warps 8-11
// softmax of tile B. TMEM: S_A, S_B (P aliases their first 64 columns), O_A, O_B = 512 columns. The 128 scores of a
// row are read in two halves (row maximum first, then exponentials) so that 384 threads fit the register file.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kAtt2Threads = 384;

struct Att2Smem {
  static constexpr int kQBytes = kQT * 256;        // one query tile, up to D = 128
  static constexpr int kKBytes = kKT * 256;
  static constexpr int kVBytes = kKT * 256;
  static constexpr int kStages = 2;
  static constexpr int kQ = 0;                     // two query tiles; each is reused as its tile's store staging
  static constexpr int kK = kQ + 2 * kQBytes;
  static constexpr int kV = kK + kStages * kKBytes;
  static constexpr int kBars = kV + kStages * kVBytes;
  static constexpr int kTotal = kBars + 256 + 1024;
};

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t* r) {
  tmem_ld32(taddr, r);
  tmem_ld32(taddr + 32, r + 32);
}

__global__ void __launch_bounds__(kAtt2Threads, 1) attention_fwd2_kernel(const __grid_constant__ AttMaps maps,
                                                                          const AttParams p) {
  constexpr int NS = Att2Smem::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Att2Smem::kBars);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;             // [NS]
  uint64_t* k_empty = k_full + NS;         // [NS]
  uint64_t* v_full = k_empty + NS;         // [NS]
  uint64_t* v_empty = v_full + NS;         // [NS]
  uint64_t* s_full = v_empty + NS;         // [2 tiles]
  uint64_t* p_full = s_full + 2;           // [2 tiles]
  uint64_t* pv_done = p_full + 2;          // [2 tiles]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = lane_id();
  const int pair_tiles = (p.q_tiles + 1) / 2;            // CTAs per group
  const int g = blockIdx.x / pair_tiles;
  const int pt = p.causal ? (pair_tiles - 1 - blockIdx.x % pair_tiles) : (blockIdx.x % pair_tiles);
  const int q0 = pt * (2 * kQT);
  // key blocks each tile needs
  const int nb_all = (p.Sk + kKT - 1) / kKT;
  int nbt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int tq0 = q0 + t * kQT;
    if (tq0 >= p.Sq) nbt[t] = 0;
    else nbt[t] = p.causal ? min(nb_all, (min(tq0 + kQT, p.Sq) - 1) / kKT + 1) : nb_all;
  }
  const int jmax = max(nbt[0], nbt[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<1>(tmem_holder, 512);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&maps.q);
    prefetch_tmap(&maps.k);
    prefetch_tmap(&maps.v);
    prefetch_tmap(&maps.o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;   // S_A 0, S_B 128, O_A 256, O_B 384

  const int d_atoms = p.D / 64, dv_chunks = p.Dv / 64;
  const uint32_t q_bytes = (uint32_t)kQT * p.D * 2, k_bytes = (uint32_t)kKT * p.D * 2, v_bytes = (uint32_t)kKT * p.Dv * 2;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * q_bytes);   // rows past the end of the sequence arrive as zeros
      for (int t = 0; t < 2; ++t)
        for (int a = 0; a < d_atoms; ++a)
          tma_load_3d(smem + Att2Smem::kQ + t * Att2Smem::kQBytes + a * (kQT * 128), &maps.q, q_full, a * 64, q0 + t * kQT, g);
      int s = 0;
      uint32_t par = 0;
      for (int j = 0; j < jmax; ++j) {
        if (!mbar_wait(&k_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + s)) break;
        uint8_t* ks = smem + Att2Smem::kK + s * Att2Smem::kKBytes;
        mbar_expect_tx(&k_full[s], k_bytes);
        if (p.trans_k) {
          for (int a = 0; a < d_atoms; ++a) tma_load_3d(ks + a * (kKT * 128), &maps.k, &k_full[s], a * 64, j * kKT, g);
        } else {
          for (int c = 0; c < kKT / 64; ++c) tma_load_3d(ks + c * (p.D * 128), &maps.k, &k_full[s], j * kKT + c * 64, 0, g);
        }
        if (!mbar_wait(&v_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + 4 + s)) break;
        uint8_t* vs = smem + Att2Smem::kV + s * Att2Smem::kVBytes;
        mbar_expect_tx(&v_full[s], v_bytes);
        for (int c = 0; c < dv_chunks; ++c) tma_load_3d(vs + c * (kKT * 128), &maps.v, &v_full[s], c * 64, j * kKT, g);
        if (++s == NS) { s = 0; par ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t hi = smem_desc_hi(1024);
      const int ksteps = p.D / 16;
      // The issuing thread must spend well under 64 cycles per 128x128x16 MMA, so every descriptor is a base
      // computed once plus a compile-time offset (loops fully unrolled, unused steps predicated off).
      const uint32_t q_lo0 = smem_desc_lo(smem_u32(smem + Att2Smem::kQ), 16);
      const uint32_t k_lo0 = p.trans_k ? smem_desc_lo(smem_u32(smem + Att2Smem::kK), 16)
                                       : smem_desc_lo(smem_u32(smem + Att2Smem::kK), (uint32_t)p.D * 128);
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(smem + Att2Smem::kV), kKT * 128);
      const uint32_t idesc_s = p.idesc_s, idesc_pv = p.idesc_pv;
      const bool trans_k = p.trans_k != 0;
      auto issue_s = [&](int t, int stage) {
        const uint32_t a_lo = q_lo0 + t * (Att2Smem::kQBytes >> 4);
        const uint32_t b_lo = k_lo0 + stage * (Att2Smem::kKBytes >> 4);
        const uint32_t d = tmem_base + t * 128;
        if (trans_k) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            if (kk < ksteps)
              umma_ss<kKindF16, 1>(d, desc64(a_lo + (((kk >> 2) * (kQT * 128) + (kk & 3) * 32) >> 4), hi),
                                   desc64(b_lo + (((kk >> 2) * (kKT * 128) + (kk & 3) * 32) >> 4), hi), idesc_s, kk ? 1u : 0u);
        } else {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            if (kk < ksteps)
              umma_ss<kKindF16, 1>(d, desc64(a_lo + (((kk >> 2) * (kQT * 128) + (kk & 3) * 32) >> 4), hi),
                                   desc64(b_lo + ((kk * 2048) >> 4), hi), idesc_s, kk ? 1u : 0u);
        }
        tc_commit<1>(&s_full[t]);
      };
      auto issue_pv = [&](int t, int stage, int j) {
        const uint32_t b_lo = v_lo0 + stage * (Att2Smem::kVBytes >> 4);
        const uint32_t tmem_p = tmem_base + t * 128;
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t acc0 = j ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kKT / 16; ++kk)
          umma_ts<kKindF16>(d, tmem_p + kk * 8, desc64(b_lo + ((kk * 2048) >> 4), hi), idesc_pv, kk ? 1u : acc0);
        tc_commit<1>(&pv_done[t]);
      };
      long long w_p[2] = {0, 0}, w_v = 0, w_k = 0;
      const long long t_begin = p.trace ? clock64() : 0;
      bool ok = mbar_wait(q_full, 0, p.status, kStatusTimeoutMma + 8);
      const long long t_q = p.trace ? clock64() : 0;
      if (ok && jmax > 0) {
        ok = mbar_wait(&k_full[0], 0, p.status, kStatusTimeoutMma + 0);
        if (ok) {
          tc_fence_after();
          if (0 < nbt[0]) issue_s(0, 0);
          if (0 < nbt[1]) issue_s(1, 0);
          tc_commit<1>(&k_empty[0]);
        }
      }
      int st = 0;          // ring stage of block j
      uint32_t par = 0;
      for (int j = 0; j < jmax && ok; ++j) {
        const int nst = (st + 1 == NS) ? 0 : st + 1;
        const uint32_t npar = (st + 1 == NS) ? (par ^ 1u) : par;
        const bool more = j + 1 < jmax;
        long long tc = p.trace ? clock64() : 0;
        if (!mbar_wait(&v_full[st], par, p.status, kStatusTimeoutMma + 10 + st)) break;
        if (p.trace) { const long long n = clock64(); w_v += n - tc; tc = n; }
        // the next K tile is waited for here, while this thread would be idle anyway, not between P.V and S of tile A
        if (more && !mbar_wait(&k_full[nst], npar, p.status, kStatusTimeoutMma + nst)) break;
        if (p.trace) { const long long n = clock64(); w_k += n - tc; tc = n; }
        if (j < nbt[0]) {
          if (!mbar_wait(&p_full[0], (uint32_t)j & 1u, p.status, kStatusTimeoutMma + 20)) break;
          if (p.trace) { const long long n = clock64(); w_p[0] += n - tc; tc = n; }
          tc_fence_after();
          issue_pv(0, st, j);
        }
        if (j + 1 < nbt[0]) issue_s(0, nst);      // S_A(j+1) overwrites S_A / P_A(j) after PV_A(j): issue order
        if (j < nbt[1]) {
          if (p.trace) tc = clock64();
          if (!mbar_wait(&p_full[1], (uint32_t)j & 1u, p.status, kStatusTimeoutMma + 21)) break;
          if (p.trace) w_p[1] += clock64() - tc;
          tc_fence_after();
          issue_pv(1, st, j);
        }
        if (j + 1 < nbt[1]) issue_s(1, nst);
        tc_commit<1>(&v_empty[st]);
        if (more) tc_commit<1>(&k_empty[nst]);
        st = nst;
        par = npar;
      }
      if (p.trace) {
        unsigned long long* tr = p.trace + (size_t)blockIdx.x * 16;
        tr[0] = (unsigned long long)(clock64() - t_begin);   // MMA thread: total
        tr[1] = (unsigned long long)(t_q - t_begin);         //   waiting for Q
        tr[2] = (unsigned long long)w_p[0];                  //   waiting for P of tile A
        tr[3] = (unsigned long long)w_p[1];                  //   waiting for P of tile B
        tr[4] = (unsigned long long)w_v;                     //   waiting for V tiles
        tr[5] = (unsigned long long)w_k;                     //   waiting for K tiles
        tr[6] = (unsigned long long)jmax;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ softmax / correction / epilogue of one tile ------------------------------
    const int t = (warp - 4) >> 2;          // tile A or B
    const int wq = warp & 3;
    const int nb = nbt[t];
    const int tq0 = q0 + t * kQT;
    const int r = wq * 32 + lane;
    const long long row = (long long)tq0 + r;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + t * 128;
    const uint32_t tmem_o = tmem_base + lane_base + 256 + t * 128;
    float m_ref = -INFINITY, l = 0.0f;
    const float qbias = p.quant_bias ? (float)*static_cast<const int8_t*>(p.quant_bias) : 0.0f;
    const float qscale = p.quant_scale ? __half2float(*static_cast<const __half*>(p.quant_scale)) : 1.0f;
    bool ok = true;
    long long sm_wait = 0, sm_busy = 0;
    for (int j = 0; j < nb && ok; ++j) {
      const long long ts0 = p.trace ? clock64() : 0;
      if (!mbar_wait(&s_full[t], (uint32_t)j & 1u, p.status, kStatusTimeoutEpilogue + t)) { ok = false; break; }
      const long long ts1 = p.trace ? clock64() : 0;
      sm_wait += ts1 - ts0;
      tc_fence_after();
      const int key0 = j * kKT;
      const bool side_inputs = p.bias || p.mask || p.scale_t || p.quant_scale;
      const bool edge = (key0 + kKT > p.Sk) || (p.causal && key0 + kKT - 1 > tq0);
      const int limit = min(p.Sk - key0, p.causal ? (int)min(row - key0 + 1, (long long)kKT) : kKT);
      const long long side_off = ((long long)g * p.Sq + min(row, (long long)p.Sq - 1)) * p.Sk + key0;
      // x(i): score of key key0 + i in the log2 domain after scale, bias and masks
      auto fx = [&](uint32_t raw, int i) -> float {
        float x = __uint_as_float(raw);
        if (p.quant_scale) {
          // Quantised form: integer-valued scores of magnitude 10^3..10^4 meet f16 steps of 1..16, so the result
          // depends on every rounding of the reference's f16 chain (cast, * quant_scale, * scale, + bias); each is
          // reproduced here before the exponent is taken in f32.
          x = f16_round(f16_round(x - qbias) * qscale);
          if (i < p.Sk - key0) {
            if (p.scale_t) x = f16_round(x * load_elem(p.scale_t, side_off + i, 0));
            if (p.bias) x = f16_round(x + load_elem(p.bias, side_off + i, 0));
            if (p.mask && p.mask[side_off + i] == 0) x = p.mask_fill;
          }
          return x * p.scale_log2;
        }
        x *= p.scale_log2;
        if (side_inputs && i < p.Sk - key0) {
          if (p.scale_t) x *= load_elem(p.scale_t, side_off + i, p.is_bf16);
          if (p.bias) x = fmaf(load_elem(p.bias, side_off + i, p.is_bf16), kLog2e, x);
          if (p.mask && p.mask[side_off + i] == 0) x = p.mask_fill * kLog2e;
        }
        return x;
      };
      if (p.linear) {
        // GEMM+GEMM: the intermediate is S itself in the element type; columns past the end of N1 are zero
        const int lim = p.Sk - key0;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t v[64];
          tmem_ld64(tmem_s + h * 64, v);
          tmem_ld_wait();
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c0 = h * 64 + 2 * i;
            w[i] = pack2((c0 < lim) ? __uint_as_float(v[2 * i]) : 0.0f, (c0 + 1 < lim) ? __uint_as_float(v[2 * i + 1]) : 0.0f, p.is_bf16);
          }
          tmem_st32(tmem_s + h * 32, w);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
        l = 1.0f;
        if (p.trace) sm_busy += clock64() - ts1;
        continue;
      }
      // pass 1: row maximum over both halves
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      float m_use = 0.0f;
      // exponent argument x(i) - m; without a bias it is the same single fused multiply-add as on the fast path, so
      // that a mask tensor and the analytic causal mask give bit-identical results
      auto fe = [&](uint32_t raw, int i) -> float {
        float a = (p.bias || p.scale_t || p.quant_scale) ? fx(raw, i) - m_use : fmaf(__uint_as_float(raw), p.scale_log2, -m_use);
        if (p.mask && i < p.Sk - key0 && p.mask[side_off + i] == 0) a = p.mask_fill * kLog2e - m_use;
        return a;
      };
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t v[64];
        tmem_ld64(tmem_s + h * 64, v);
        tmem_ld_wait();
        if (!side_inputs && !edge) {
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(v[i])); mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(v[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
          }
        } else if (!side_inputs) {
          // key tail / diagonal block: keys at or past `limit` are dropped with a select
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            const int c0 = h * 64 + i;
            mx0 = fmaxf(mx0, (c0 < limit) ? __uint_as_float(v[i]) : -INFINITY);
            mx1 = fmaxf(mx1, (c0 + 1 < limit) ? __uint_as_float(v[i + 1]) : -INFINITY);
            mx2 = fmaxf(mx2, (c0 + 2 < limit) ? __uint_as_float(v[i + 2]) : -INFINITY);
            mx3 = fmaxf(mx3, (c0 + 3 < limit) ? __uint_as_float(v[i + 3]) : -INFINITY);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float x = (h * 64 + i < limit) ? fx(v[i], h * 64 + i) : -INFINITY;
            mx0 = fmaxf(mx0, x);
          }
        }
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      if (!side_inputs) mx *= p.scale_log2;   // the scale is positive: max commutes with it (-inf stays -inf)
      float alpha = 1.0f;
      if (mx > m_ref + 8.0f || (m_ref == -INFINITY && mx > -INFINITY)) {
        alpha = ex2(m_ref - mx);
        m_ref = mx;
      }
      m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
      // pass 2: exponentials, row sum, P over the first 64 columns of the score buffer
      float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t v[64];
        tmem_ld64(tmem_s + h * 64, v);
        tmem_ld_wait();
        uint32_t w[32];
        if (!side_inputs && !edge) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, -m_use));
            const float p1 = ex2(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, -m_use));
            const float p2 = ex2(fmaf(__uint_as_float(v[2 * i + 2]), p.scale_log2, -m_use));
            const float p3 = ex2(fmaf(__uint_as_float(v[2 * i + 3]), p.scale_log2, -m_use));
            l0 += p0; l1 += p1; l2 += p2; l3 += p3;
            w[i] = pack2(p0, p1, p.is_bf16);
            w[i + 1] = pack2(p2, p3, p.is_bf16);
          }
        } else if (!side_inputs) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int c0 = h * 64 + 2 * i;
            const float p0 = (c0 < limit) ? ex2(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, -m_use)) : 0.0f;
            const float p1 = (c0 + 1 < limit) ? ex2(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, -m_use)) : 0.0f;
            const float p2 = (c0 + 2 < limit) ? ex2(fmaf(__uint_as_float(v[2 * i + 2]), p.scale_log2, -m_use)) : 0.0f;
            const float p3 = (c0 + 3 < limit) ? ex2(fmaf(__uint_as_float(v[2 * i + 3]), p.scale_log2, -m_use)) : 0.0f;
            l0 += p0; l1 += p1; l2 += p2; l3 += p3;
            w[i] = pack2(p0, p1, p.is_bf16);
            w[i + 1] = pack2(p2, p3, p.is_bf16);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c0 = h * 64 + 2 * i;
            const float p0 = (c0 < limit) ? ex2(fe(v[2 * i], c0)) : 0.0f;
            const float p1 = (c0 + 1 < limit) ? ex2(fe(v[2 * i + 1], c0 + 1)) : 0.0f;
            if (i & 1) { l2 += p0; l3 += p1; } else { l0 += p0; l1 += p1; }   // same summation order as the fast path
            w[i] = pack2(p0, p1, p.is_bf16);
          }
        }
        // half h of P -> columns 32h .. 32h+31 (both halves of S are in registers or consumed by now only for
        // h = 1; for h = 0 the columns 0..31 written here belong to the half already read)
        tmem_st32(tmem_s + h * 32, w);
      }
      l = l * alpha + ((l0 + l1) + (l2 + l3));
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        if (!mbar_wait(&pv_done[t], (uint32_t)(j - 1) & 1u, p.status, kStatusTimeoutEpilogue + 4 + t)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < p.Dv / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_o + c * 32, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      if (p.trace) sm_busy += clock64() - ts1;
    }
    if (p.trace && wq == 0 && lane == 0) {
      p.trace[(size_t)blockIdx.x * 16 + 8 + 2 * t] = (unsigned long long)sm_wait;   // softmax group t: waiting for S
      p.trace[(size_t)blockIdx.x * 16 + 9 + 2 * t] = (unsigned long long)sm_busy;   //   busy (incl. rescale)
    }
    if (ok && nb > 0 && mbar_wait(&pv_done[t], (uint32_t)(nb - 1) & 1u, p.status, kStatusTimeoutEpilogue + 6 + t)) {
      tc_fence_after();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      uint8_t* stg = smem + Att2Smem::kQ + t * Att2Smem::kQBytes + wq * (2 * 32 * 128);
#pragma unroll 1
      for (int c = 0; c < p.Dv / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + c * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, p.is_bf16);
        uint8_t* rowp = stg + (c >> 1) * (32 * 128) + lane * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int piece = (c & 1) * 4 + i;
          *reinterpret_cast<uint4*>(rowp + ((piece ^ (lane & 7)) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0 && tq0 + wq * 32 < p.Sq) {
        for (int c = 0; c < p.Dv / 64; ++c) tma_store_3d(&maps.o, stg + c * (32 * 128), c * 64, tq0 + wq * 32, g);
        bulk_commit();
        bulk_wait<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// i8 -> f16 (exact) for the first-GEMM-quantised form: 16 elements per thread where the count allows
__global__ void widen_i8_kernel(const int8_t* __restrict__ src, __half* __restrict__ dst, long long n) {
  const long long nv = (reinterpret_cast<uintptr_t>(src) % 16 == 0) ? n / 16 : 0;   // vector part needs an aligned source
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const int4 raw = reinterpret_cast<const int4*>(src)[i];
    const int w[4] = {raw.x, raw.y, raw.z, raw.w};
    __half2 out[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] = __floats2half2_rn((float)(int8_t)(w[j] & 0xff), (float)(int8_t)((w[j] >> 8) & 0xff));
      out[2 * j + 1] = __floats2half2_rn((float)(int8_t)((w[j] >> 16) & 0xff), (float)(int8_t)((w[j] >> 24) & 0xff));
    }
    reinterpret_cast<int4*>(dst)[2 * i] = *reinterpret_cast<int4*>(&out[0]);
    reinterpret_cast<int4*>(dst)[2 * i + 1] = *reinterpret_cast<int4*>(&out[4]);
  }
  for (long long i = nv * 16 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2half_rn((float)src[i]);
}

// dst[g][r][c] (row pitch dst_pitch) = src[g * s_g + r * s_r + c * s_c] for 2-byte elements: the transposed operand
// forms (transQ / transV / transO of rocmlir-gen) and K rows that do not start on 16-byte boundaries are brought to
// the layout the kernels load, in scratch memory. Consecutive threads walk c, so the destination is written in rows.
__global__ void restride16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, long long G, long long R,
                                  long long C, long long dst_pitch, long long s_g, long long s_r, long long s_c) {
  const long long total = G * R * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i % C, t = i / C;
    const long long r = t % R, g = t / R;
    dst[(g * R + r) * dst_pitch + c] = src[g * s_g + r * s_r + c * s_c];
  }
}

// f32 attention is a precision-first path. The reference's f32 suite accepts a relative difference of 5e-6 on EVERY
// nonzero element (PrAttentionF32.toml:3), including results that are small by cancellation; a TF32 split (hi + lo,
// 22 bits) leaves 5e-7 of the largest term there, which fails it, so both products run in true f32 on the FMA pipe
// (sgemm_strided_kernel) around this row softmax over the score matrix in scratch. Operation order is the
// reference's (rocmlir-gen.cpp:2582-2630): f(s), row maximum, exp(s - max), row sum, times the reciprocal of the sum.
struct SgemmParams {
  int M, N, K;
  long long a_g, a_m, a_k;   // element strides of A[g][m][k], B[g][k][n], C[g][m][n]
  long long b_g, b_k, b_n;
  long long c_g, c_m, c_n;
};

// C = A . B in f32, k ascending, product and sum rounded separately like the reference's generated host loops (no
// contraction flags are set there): 64 x 64 tile per 256-thread block, 4 x 4 per thread
__global__ void __launch_bounds__(256) sgemm_strided_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                            float* __restrict__ C, SgemmParams p) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const float* Ag = A + (long long)blockIdx.z * p.a_g;
  const float* Bg = B + (long long)blockIdx.z * p.b_g;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < p.K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      // A tile: walk the dimension that is contiguous in memory fastest
      const int am = p.a_k == 1 ? idx / 16 : idx % 64, ak = p.a_k == 1 ? idx % 16 : idx / 64;
      As[ak][am] = (m0 + am < p.M && k0 + ak < p.K) ? Ag[(long long)(m0 + am) * p.a_m + (long long)(k0 + ak) * p.a_k] : 0.0f;
      const int bn = p.b_n == 1 ? idx % 64 : idx / 16, bk = p.b_n == 1 ? idx / 64 : idx % 16;
      Bs[bk][bn] = (n0 + bn < p.N && k0 + bk < p.K) ? Bg[(long long)(k0 + bk) * p.b_k + (long long)(n0 + bn) * p.b_n] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));   // no contraction
    }
    __syncthreads();
  }
  float* Cg = C + (long long)blockIdx.z * p.c_g;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < p.M && n < p.N) Cg[(long long)m * p.c_m + (long long)n * p.c_n] = acc[i][j];
    }
}

struct SoftmaxF32Params {
  long long G, Sq, Sk;
  int has_scale, causal;
  float scale, mask_fill;
  const float* scale_t;
  const float* bias;
  const int8_t* mask;
};

__global__ void softmax_rows_f32_kernel(float* __restrict__ s, SoftmaxF32Params p) {
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  auto block_reduce = [&](float v, bool is_max) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float w = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, w) : v + w;
    }
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < nwarps; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    return r;
  };
  for (long long row = blockIdx.x; row < p.G * p.Sq; row += gridDim.x) {
    float* sr = s + row * p.Sk;
    const long long q = row % p.Sq;
    const long long side = row * p.Sk;
    float mx = -INFINITY;
    for (long long j = threadIdx.x; j < p.Sk; j += blockDim.x) {
      float x = sr[j];
      if (p.has_scale) x *= p.scale;
      if (p.scale_t) x *= p.scale_t[side + j];
      if (p.bias) x += p.bias[side + j];
      if (p.mask && p.mask[side + j] == 0) x = p.mask_fill;
      if (p.causal && j > q) x = -INFINITY;
      sr[j] = x;
      mx = fmaxf(mx, x);
    }
    mx = block_reduce(mx, true);
    // exp through double and rounded once (what the host's expf returns), and the row sum taken by one thread in key
    // order like the reference's loop: results that are small by cancellation inherit every ulp of P, and the f32
    // suite judges each element at 5e-6 relative
    for (long long j = threadIdx.x; j < p.Sk; j += blockDim.x)
      sr[j] = (mx == -INFINITY) ? 0.0f : (float)exp((double)(sr[j] - mx));
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.0f;
      for (long long j = 0; j < p.Sk; ++j) acc = __fadd_rn(acc, sr[j]);
      red[0] = acc;
    }
    __syncthreads();
    const float l = red[0];
    const float rl = l > 0.0f ? 1.0f / l : 0.0f;
    for (long long j = threadIdx.x; j < p.Sk; j += blockDim.x) sr[j] *= rl;
  }
}

// Scratch for the widened Q and K: grow-only, owned by the calling thread (a growth waits for the device first, so
// no kernel in flight still reads the old block).
struct QkScratch {
  void* ptr = nullptr;
  size_t size = 0;
  int device = -1;
};
thread_local QkScratch t_qk;

RbStatus qk_reserve(size_t bytes) {
  int dev = 0;
  RB_CUDA_TRY(cudaGetDevice(&dev));
  if (t_qk.device == dev && t_qk.size >= bytes) return RB_SUCCESS;
  if (t_qk.ptr) {
    RB_CUDA_TRY(cudaDeviceSynchronize());
    RB_CUDA_TRY(cudaFree(t_qk.ptr));
    t_qk = QkScratch();
  }
  RB_CUDA_TRY(cudaMalloc(&t_qk.ptr, bytes));
  t_qk.size = bytes;
  t_qk.device = dev;
  return RB_SUCCESS;
}

RbStatus attention_f32(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o, void* scratch,
                       void* stream_v) {
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const long long G = p->g, Sq = p->seq_q, Sk = p->seq_k, D = p->head_qk, Dv = p->head_v;
  if (G > 65535) return fail(RB_UNSUPPORTED, "f32 attention: more than 65535 groups");
  float* s = static_cast<float*>(scratch);
  SgemmParams g1;   // S[g] = Q[g] . K[g]:  M = Sq, N = Sk, K = D
  g1.M = (int)Sq; g1.N = (int)Sk; g1.K = (int)D;
  g1.a_g = Sq * D; g1.a_m = p->trans_q ? 1 : D; g1.a_k = p->trans_q ? Sq : 1;     // Q [Sq][D] or [D][Sq]
  g1.b_g = Sk * D; g1.b_k = p->trans_k ? 1 : Sk; g1.b_n = p->trans_k ? D : 1;     // K [D][Sk] or [Sk][D]
  g1.c_g = Sq * Sk; g1.c_m = Sk; g1.c_n = 1;
  sgemm_strided_kernel<<<dim3((unsigned)((Sk + 63) / 64), (unsigned)((Sq + 63) / 64), (unsigned)G), 256, 0, stream>>>(
      static_cast<const float*>(q), static_cast<const float*>(k), s, g1);
  SoftmaxF32Params sp;
  sp.G = G; sp.Sq = Sq; sp.Sk = Sk;
  sp.has_scale = p->has_scale; sp.causal = p->causal; sp.scale = p->scale; sp.mask_fill = p->mask_fill;
  sp.scale_t = static_cast<const float*>(p->scale_tensor);
  sp.bias = static_cast<const float*>(p->bias);
  sp.mask = p->mask;
  softmax_rows_f32_kernel<<<(unsigned)std::min<long long>(G * Sq, (long long)dev->sm_count * 16), 256, 0, stream>>>(s, sp);
  SgemmParams g2;   // O[g] = P[g] . V[g]:  M = Sq, N = Dv, K = Sk
  g2.M = (int)Sq; g2.N = (int)Dv; g2.K = (int)Sk;
  g2.a_g = Sq * Sk; g2.a_m = Sk; g2.a_k = 1;
  g2.b_g = Sk * Dv; g2.b_k = p->trans_v ? 1 : Dv; g2.b_n = p->trans_v ? Sk : 1;   // V [Sk][Dv] or [Dv][Sk]
  g2.c_g = Sq * Dv; g2.c_m = p->trans_o ? 1 : Dv; g2.c_n = p->trans_o ? Sq : 1;   // O [Sq][Dv] or [Dv][Sq]
  sgemm_strided_kernel<<<dim3((unsigned)((Dv + 63) / 64), (unsigned)((Sq + 63) / 64), (unsigned)G), 256, 0, stream>>>(
      s, static_cast<const float*>(v), static_cast<float*>(o), g2);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch(3);
  return RB_SUCCESS;
}

// Scratch an attention call stages operands in (0 for the plain f16 / bf16 form with loadable layouts).
struct AttScratch {
  size_t qw_off, kw_off, qt_off, kp_off, vt_off, ot_off, total;
  long long sk_pitch;
  bool k_repitch;
};
AttScratch plan_scratch(const RbAttentionProblem* p) {
  AttScratch a{};
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  if (p->data_type == RB_F32) {   // the whole score matrix
    a.total = up((size_t)p->g * p->seq_q * p->seq_k * 4);
    return a;
  }
  const bool quantized = p->data_type == RB_I8;
  const size_t qn = (size_t)p->g * p->seq_q * p->head_qk, kn = (size_t)p->g * p->seq_k * p->head_qk;
  const size_t vn = (size_t)p->g * p->seq_k * p->head_v, on = (size_t)p->g * p->seq_q * p->head_v;
  a.sk_pitch = (p->seq_k + 7) / 8 * 8;
  a.k_repitch = !p->trans_k && p->seq_k % 8 != 0;
  size_t off = 0;
  a.qw_off = off; off += quantized ? up(qn * 2) : 0;
  a.kw_off = off; off += quantized ? up(kn * 2) : 0;
  a.qt_off = off; off += p->trans_q ? up(qn * 2) : 0;
  a.kp_off = off; off += a.k_repitch ? up((size_t)p->g * p->head_qk * a.sk_pitch * 2) : 0;
  a.vt_off = off; off += p->trans_v ? up(vn * 2) : 0;
  a.ot_off = off; off += p->trans_o ? up(on * 2) : 0;
  a.total = off;
  return a;
}
bool valid_sizes(const RbAttentionProblem* p) {
  return p && p->g > 0 && p->seq_q > 0 && p->seq_k > 0 && p->head_qk > 0 && p->head_v > 0;
}
}  // namespace
static RbStatus attention_run(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o,
                              void* workspace, size_t workspace_bytes, bool own_scratch, void* stream_v);
}  // namespace rb

using namespace rb;

extern "C" size_t rbAttentionWorkspaceSize(const RbAttentionProblem* p) {
  return valid_sizes(p) ? plan_scratch(p).total : 0;
}

extern "C" RbStatus rbAttentionWs(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o,
                                  void* workspace, size_t workspace_bytes, void* stream_v) {
  return attention_run(p, q, k, v, o, workspace, workspace_bytes, false, stream_v);
}

extern "C" RbStatus rbAttention(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o,
                                void* stream_v) {
  return attention_run(p, q, k, v, o, nullptr, 0, true, stream_v);
}

namespace rb {
static thread_local bool t_attention_linear = false;

// O = (A . B1) . B2 on the attention kernels with the softmax taken out: A [g][m][k1] as Q, B1 [g][k1][n1] as K,
// B2 [g][n1][n2] as V; the intermediate never leaves the SM (S in tensor memory -> rounded to the element type in
// place -> A operand of the second product). k1 and n2 at most 128 (the kernels' head dimensions).
bool gemm_gemm_on_chip_applicable(int32_t k1, int32_t n1, int32_t n2, int32_t data_type) {
  return (data_type == RB_F16 || data_type == RB_BF16) && k1 % 8 == 0 && k1 <= 128 && n2 % 8 == 0 && n2 <= 128 && n1 % 8 == 0;
}
RbStatus gemm_gemm_on_chip(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type, const void* a,
                           const void* b1, const void* b2, void* o, void* stream) {
  RbAttentionProblem p;
  memset(&p, 0, sizeof(p));
  p.g = g; p.seq_q = m; p.seq_k = n1; p.head_qk = k1; p.head_v = n2; p.data_type = data_type;
  t_attention_linear = true;
  const RbStatus st = attention_run(&p, a, b1, b2, o, nullptr, 0, false, stream);
  t_attention_linear = false;
  return st;
}
}  // namespace rb

static RbStatus rb::attention_run(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o,
                                  void* workspace, size_t workspace_bytes, bool own_scratch, void* stream_v) {
  if (!p) return fail(RB_INVALID_PARAM, "problem is NULL");
  if (p->g <= 0 || p->seq_q <= 0 || p->seq_k <= 0 || p->head_qk <= 0 || p->head_v <= 0)
    return fail(RB_INVALID_PARAM, "g, seq_len_q, seq_len_k, head_dim_qk, head_dim_v must be positive");
  if (!q || !k || !v || !o) return fail(RB_INVALID_PARAM, "q, k, v and o must be device pointers");
  const bool quantized = p->data_type == RB_I8;
  const AttScratch sc = plan_scratch(p);
  uint8_t* base = nullptr;
  if (sc.total) {
    if (own_scratch) {       // rbAttention: the calling thread's grow-only block (allocates on growth)
      RbStatus st = qk_reserve(sc.total);
      if (st != RB_SUCCESS) return st;
      base = static_cast<uint8_t*>(t_qk.ptr);
    } else {
      if (!workspace || workspace_bytes < sc.total)
        return fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(sc.total) + " bytes required");
      if (reinterpret_cast<uintptr_t>(workspace) % 16) return fail(RB_INVALID_PARAM, "workspace must be 16-byte aligned");
      base = static_cast<uint8_t*>(workspace);
    }
  }
  if (p->data_type == RB_F32) return attention_f32(p, q, k, v, o, base, stream_v);
  if (!(p->data_type == RB_F16 || p->data_type == RB_BF16 || quantized))
    return fail(RB_UNSUPPORTED, "attention exists for f32, f16, bf16 and the first-GEMM-quantised i8 form");
  if (quantized && (!p->quant_bias || !p->quant_scale))
    return fail(RB_INVALID_PARAM, "the i8 form needs quant_bias and quant_scale");
  if (quantized && p->causal) return fail(RB_UNSUPPORTED, "the i8 form has no analytic causal mask");
  // Head dimensions that are not 64 or 128 run as the next multiple of 64: the TMA boxes are 64 elements wide, what
  // they cover beyond the tensor arrives as zeros (no contribution to Q.K, zero columns of O) and is clipped on the
  // store of O. A row of Q, K, V or O must still start on a 16-byte boundary.
  if (p->head_qk % 8 || p->head_qk > 128 || p->head_v % 8 || p->head_v > 128)
    return fail(RB_UNSUPPORTED, "head dimensions must be multiples of 8, at most 128");
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  // Operands the kernels cannot load as they lie are staged in scratch the calling thread owns: i8 Q and K widened
  // to f16 (every value and product exact; the f32 accumulation of at most 128 * 127 * 127 stays below 2^24, so the
  // score equals the reference's i32), Q / V stored transposed, K stored G x D x Sk with rows off 16-byte boundaries;
  // a transposed O is written to scratch and turned afterwards.
  const size_t qn = (size_t)p->g * p->seq_q * p->head_qk, kn = (size_t)p->g * p->seq_k * p->head_qk;
  const long long sk_pitch = sc.sk_pitch;
  const bool k_repitch = sc.k_repitch;
  const size_t qw_off = sc.qw_off, kw_off = sc.kw_off, qt_off = sc.qt_off, kp_off = sc.kp_off, vt_off = sc.vt_off,
               ot_off = sc.ot_off;
  const int sblocks = dev->sm_count * 8;
  if (quantized) {
    widen_i8_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const int8_t*>(q), reinterpret_cast<__half*>(base + qw_off), (long long)qn);
    widen_i8_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const int8_t*>(k), reinterpret_cast<__half*>(base + kw_off), (long long)kn);
    count_launch(2);
    q = base + qw_off;
    k = base + kw_off;
  }
  if (p->trans_q) {   // stored [G][D][Sq]
    restride16_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const uint16_t*>(q), reinterpret_cast<uint16_t*>(base + qt_off), p->g,
                                                   p->seq_q, p->head_qk, p->head_qk, (long long)p->head_qk * p->seq_q, 1, p->seq_q);
    count_launch();
    q = base + qt_off;
  }
  if (k_repitch) {    // stored [G][D][Sk]: the same with a row pitch of a multiple of 8 elements
    restride16_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const uint16_t*>(k), reinterpret_cast<uint16_t*>(base + kp_off), p->g,
                                                   p->head_qk, p->seq_k, sk_pitch, (long long)p->head_qk * p->seq_k, p->seq_k, 1);
    count_launch();
    k = base + kp_off;
  }
  if (p->trans_v) {   // stored [G][Dv][Sk]
    restride16_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const uint16_t*>(v), reinterpret_cast<uint16_t*>(base + vt_off), p->g,
                                                   p->seq_k, p->head_v, p->head_v, (long long)p->head_v * p->seq_k, 1, p->seq_k);
    count_launch();
    v = base + vt_off;
  }
  void* o_user = o;
  if (p->trans_o) o = base + ot_off;
  AttMaps maps;
  memset(&maps, 0, sizeof(maps));
  const CUtensorMapDataType dt = p->data_type == RB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  std::string err;
  const uint64_t G = p->g, Sq = p->seq_q, Sk = p->seq_k, D = p->head_qk, Dv = p->head_v;
  const uint64_t Dp = (D + 63) / 64 * 64, Dvp = (Dv + 63) / 64 * 64;   // extents the kernels work on
  {
    const uint64_t dims[3] = {D, Sq, G};
    const uint64_t str[2] = {D * 2, Sq * D * 2};
    const uint32_t box[3] = {64, (uint32_t)kQT, 1};
    if (!encode_tiled(&maps.q, dt, 3, q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, &err)) return fail(RB_UNSUPPORTED, "Q: " + err);
  }
  if (p->trans_k) {
    const uint64_t dims[3] = {D, Sk, G};
    const uint64_t str[2] = {D * 2, Sk * D * 2};
    const uint32_t box[3] = {64, (uint32_t)kKT, 1};
    if (!encode_tiled(&maps.k, dt, 3, k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, &err)) return fail(RB_UNSUPPORTED, "K: " + err);
  } else {
    const uint64_t dims[3] = {Sk, D, G};
    const uint64_t pitch = k_repitch ? (uint64_t)sk_pitch : Sk;
    const uint64_t str[2] = {pitch * 2, D * pitch * 2};
    const uint32_t box[3] = {64, (uint32_t)Dp, 1};
    if (!encode_tiled(&maps.k, dt, 3, k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, &err)) return fail(RB_UNSUPPORTED, "K: " + err);
  }
  {
    const uint64_t dims[3] = {Dv, Sk, G};
    const uint64_t str[2] = {Dv * 2, Sk * Dv * 2};
    const uint32_t box[3] = {64, (uint32_t)kKT, 1};
    if (!encode_tiled(&maps.v, dt, 3, v, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, &err)) return fail(RB_UNSUPPORTED, "V: " + err);
  }
  {
    const uint64_t dims[3] = {Dv, Sq, G};
    const uint64_t str[2] = {Dv * 2, Sq * Dv * 2};
    const uint32_t box[3] = {64, 32, 1};
    if (!encode_tiled(&maps.o, dt, 3, o, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, &err)) return fail(RB_UNSUPPORTED, "O: " + err);
  }
  AttParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.G = p->g; kp.Sq = p->seq_q; kp.Sk = p->seq_k; kp.D = (int)Dp; kp.Dv = (int)Dvp;
  kp.trans_k = p->trans_k ? 1 : 0;
  kp.is_bf16 = p->data_type == RB_BF16;
  kp.causal = p->causal ? 1 : 0;
  kp.q_tiles = (p->seq_q + kQT - 1) / kQT;
  kp.scale_log2 = (p->has_scale ? p->scale : 1.0f) * kLog2e;
  kp.bias = p->bias;
  kp.scale_t = p->scale_tensor;
  kp.quant_bias = quantized ? p->quant_bias : nullptr;
  kp.quant_scale = quantized ? p->quant_scale : nullptr;
  kp.mask = p->mask;
  kp.mask_fill = p->mask_fill;
  kp.linear = t_attention_linear ? 1 : 0;
  const uint32_t fmt = kp.is_bf16 ? 1u : 0u;
  kp.idesc_s = make_idesc(1, fmt, fmt, 0, p->trans_k ? 0u : 1u, kQT, kKT);
  kp.idesc_pv = make_idesc(1, fmt, fmt, 0, 1u, kQT, (uint32_t)Dvp);
  kp.status = dev->status_word;
  kp.trace = trace_buffer((size_t)p->g * ((kp.q_tiles + 1) / 2) * 16);
  const long long ctas = (long long)p->g * kp.q_tiles;
  if (ctas > 0x7fffffffLL) return fail(RB_UNSUPPORTED, "too many query tiles");
  const float eff_scale = p->has_scale ? p->scale : 1.0f;   // an unset scale field must not pick the kernel
  if (p->seq_q > kQT && eff_scale >= 0.0f) {
    // two query tiles per CTA (the fast path folds the scale into the row maximum, which needs scale >= 0)
    const long long ctas2 = (long long)p->g * ((kp.q_tiles + 1) / 2);
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(attention_fwd2_kernel), Att2Smem::kTotal) != RB_SUCCESS) return RB_CUDA_ERROR;
    attention_fwd2_kernel<<<(unsigned)ctas2, kAtt2Threads, Att2Smem::kTotal, stream>>>(maps, kp);
  } else {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(attention_fwd_kernel), AttSmem::kTotal) != RB_SUCCESS) return RB_CUDA_ERROR;
    attention_fwd_kernel<<<(unsigned)ctas, kAttThreads, AttSmem::kTotal, stream>>>(maps, kp);
  }
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  if (p->trans_o) {   // caller's O is [G][Dv][Sq]
    restride16_kernel<<<sblocks, 256, 0, stream>>>(static_cast<const uint16_t*>(o), static_cast<uint16_t*>(o_user), p->g, p->head_v,
                                                   p->seq_q, p->seq_q, (long long)p->seq_q * p->head_v, 1, p->head_v);
    RB_CUDA_TRY(cudaGetLastError());
    count_launch();
  }
  return RB_SUCCESS;
}
