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
// CTA = one 128-row query tile, 256 threads:
//   warp 0   producer: TMA loads of Q (once) and of the K and V tiles of each key block (2-deep rings)
//   warp 1   MMA issuer: S_j = Q.K_j^T into one of two TMEM score buffers, O += P_j.V_j
//   warp 2   TMEM allocator
//   warps 4-7 softmax: thread = query row (TMEM lane). Two passes over the score tile in TMEM (row max, then
//            exp2 / row sum / P in f16 written to 128-byte-swizzled shared memory as the A operand of P.V),
//            rescale of O in TMEM when a row maximum moved, final O / l and TMA store.
// S_{j+1} is issued before P_j is awaited, so the score MMA of the next block overlaps the softmax of this one.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

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
  const int8_t* mask;  // optional [G][Sq][Sk]: score kept where mask != 0, else mask_fill
  float mask_fill;
  uint32_t idesc_s, idesc_pv;
  uint32_t* status;
};

struct AttSmem {
  static constexpr int kQBytes = kQT * 256;        // up to D = 128 f16
  static constexpr int kKBytes = kKT * 256;
  static constexpr int kVBytes = kKT * 256;
  static constexpr int kPBytes = kQT * kKT * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQBytes;          // 2 stages
  static constexpr int kV = kK + 2 * kKBytes;      // 2 stages
  static constexpr int kP = kV + 2 * kVBytes;
  static constexpr int kBars = kP + kPBytes;
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

__global__ void __launch_bounds__(kAttThreads, 1) attention_fwd_kernel(const __grid_constant__ AttMaps maps,
                                                                        const AttParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::kBars);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_free = bars + 11;   // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 16);

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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
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
  const uint32_t tmem_o = tmem_base + 256;

  const int d_atoms = p.D / 64, dv_chunks = p.Dv / 64;
  const uint32_t q_bytes = (uint32_t)kQT * p.D * 2, k_bytes = (uint32_t)kKT * p.D * 2, v_bytes = (uint32_t)kKT * p.Dv * 2;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, q_bytes);
      for (int a = 0; a < d_atoms; ++a) tma_load_3d(smem + AttSmem::kQ + a * (kQT * 128), &maps.q, q_full, a * 64, q0, g);
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        const uint32_t par = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(&k_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + s)) break;
        uint8_t* ks = smem + AttSmem::kK + s * AttSmem::kKBytes;
        mbar_expect_tx(&k_full[s], k_bytes);
        if (p.trans_k) {
          for (int a = 0; a < d_atoms; ++a) tma_load_3d(ks + a * (kKT * 128), &maps.k, &k_full[s], a * 64, j * kKT, g);
        } else {
          for (int c = 0; c < kKT / 64; ++c) tma_load_3d(ks + c * (p.D * 128), &maps.k, &k_full[s], j * kKT + c * 64, 0, g);
        }
        if (!mbar_wait(&v_empty[s], par ^ 1u, p.status, kStatusTimeoutProducer + 2 + s)) break;
        uint8_t* vs = smem + AttSmem::kV + s * AttSmem::kVBytes;
        mbar_expect_tx(&v_full[s], v_bytes);
        for (int c = 0; c < dv_chunks; ++c) tma_load_3d(vs + c * (kKT * 128), &maps.v, &v_full[s], c * 64, j * kKT, g);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t hi = smem_desc_hi(1024);
      const uint32_t q_addr = smem_u32(smem + AttSmem::kQ), p_addr = smem_u32(smem + AttSmem::kP);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (uint32_t)(j >> 1) & 1u, p.status, kStatusTimeoutMma + s)) return false;
        if (!mbar_wait(&s_free[s], ((uint32_t)(j >> 1) & 1u) ^ 1u, p.status, kStatusTimeoutMma + 4 + s)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + AttSmem::kK + s * AttSmem::kKBytes);
        const int ksteps = p.D / 16;
        for (int kk = 0; kk < ksteps; ++kk) {
          const uint32_t a_lo = smem_desc_lo(q_addr + (kk >> 2) * (kQT * 128) + (kk & 3) * 32, 16);
          const uint32_t b_lo = p.trans_k ? smem_desc_lo(k_addr + (kk >> 2) * (kKT * 128) + (kk & 3) * 32, 16)
                                          : smem_desc_lo(k_addr + kk * 2048, (uint32_t)p.D * 128);
          umma_ss<kKindF16, 1>(tmem_base + s * 128, desc64(a_lo, hi), desc64(b_lo, hi), p.idesc_s, kk ? 1u : 0u);
        }
        tc_commit<1>(&s_full[s]);
        tc_commit<1>(&k_empty[s]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, p.status, kStatusTimeoutMma + 8);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        if (!mbar_wait(p_full, (uint32_t)j & 1u, p.status, kStatusTimeoutMma + 9)) break;
        if (!mbar_wait(&v_full[s], (uint32_t)(j >> 1) & 1u, p.status, kStatusTimeoutMma + 10 + s)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + AttSmem::kV + s * AttSmem::kVBytes);
        for (int kk = 0; kk < kKT / 16; ++kk) {
          const uint32_t a_lo = smem_desc_lo(p_addr + (kk >> 2) * (kQT * 128) + (kk & 3) * 32, 16);
          const uint32_t b_lo = smem_desc_lo(v_addr + kk * 2048, kKT * 128);
          umma_ss<kKindF16, 1>(tmem_o, desc64(a_lo, hi), desc64(b_lo, hi), p.idesc_pv, (j | kk) ? 1u : 0u);
        }
        tc_commit<1>(pv_done);
        tc_commit<1>(&v_empty[s]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int wq = warp & 3;
    const int r = wq * 32 + lane;          // row within the tile == TMEM lane
    const long long row = (long long)q0 + r;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    uint8_t* p_smem = smem + AttSmem::kP;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < nb && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], (uint32_t)(j >> 1) & 1u, p.status, kStatusTimeoutEpilogue + s)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_s = tmem_base + lane_base + s * 128;
      const int key0 = j * kKT;
      const bool need_mask = (key0 + kKT > p.Sk) || (p.causal && key0 + kKT - 1 > q0) || p.bias || p.mask;
      const long long side_off = ((long long)g * p.Sq + min(row, (long long)p.Sq - 1)) * p.Sk;
      // f(S): scale, bias, masks; returns the score in the log2 domain
      auto score = [&](uint32_t raw, int col) -> float {
        float x = __uint_as_float(raw) * p.scale_log2;
        if (need_mask) {
          const int key = key0 + col;
          if (key < p.Sk) {
            if (p.bias) x = fmaf(load_elem(p.bias, side_off + key, p.is_bf16), kLog2e, x);
            if (p.mask && p.mask[side_off + key] == 0) x = p.mask_fill * kLog2e;
            if (p.causal && key > row) x = -INFINITY;
          } else {
            x = -INFINITY;
          }
        }
        return x;
      };
      // pass 1: row maximum
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, score(v[i], c * 32 + i));
      }
      const float m_use = (mx == -INFINITY) ? 0.0f : mx;   // a fully masked row keeps exp2 finite
      const float alpha = exp2f(m - m_use);                  // m = -inf on the first block -> 0
      // the P buffer and O are free once P_{j-1}.V_{j-1} has completed
      if (j > 0 && !mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, p.status, kStatusTimeoutEpilogue + 4)) { ok = false; break; }
      // pass 2: p = exp2(x - m), row sum, P (element type) into the swizzled A-operand tile
      float lsum = 0.0f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + c * 32, v);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(score(v[2 * i], c * 32 + 2 * i) - m_use);
          const float p1 = exp2f(score(v[2 * i + 1], c * 32 + 2 * i + 1) - m_use);
          lsum += p0 + p1;
          w[i] = pack2(p0, p1, p.is_bf16);
        }
        // 32 keys = 64 bytes = 4 pieces of 16 bytes; atom = 64 keys
        uint8_t* rowp = p_smem + (c >> 1) * (kQT * 128) + r * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int piece = (c & 1) * 4 + i;
          *reinterpret_cast<uint4*>(rowp + ((piece ^ (r & 7)) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      // the score buffer may be overwritten by S_{j+2}
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);
      l = l * alpha + lsum;
      m = mx;
      // rescale O where a row maximum moved (whole warp takes part: TMEM access is warp-collective)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < p.Dv / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_base + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st32(tmem_o + lane_base + c * 32, v);
        }
        tmem_st_wait();
      }
      fence_proxy_async();   // P written through the generic proxy, read by the MMA through the async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> element type -> staging (the P tile is free now) -> TMA store ----
    if (ok && mbar_wait(pv_done, (uint32_t)(nb - 1) & 1u, p.status, kStatusTimeoutEpilogue + 5)) {
      tc_fence_after();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      uint8_t* stg = p_smem + wq * (2 * 32 * 128);   // per warp: Dv/64 tiles of 32 rows x 128 bytes
#pragma unroll 1
      for (int c = 0; c < p.Dv / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_base + c * 32, v);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv, p.is_bf16);
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

}  // namespace
}  // namespace rb

using namespace rb;

extern "C" RbStatus rbAttention(const RbAttentionProblem* p, const void* q, const void* k, const void* v, void* o,
                                void* stream_v) {
  if (!p) return fail(RB_INVALID_PARAM, "problem is NULL");
  if (p->g <= 0 || p->seq_q <= 0 || p->seq_k <= 0 || p->head_qk <= 0 || p->head_v <= 0)
    return fail(RB_INVALID_PARAM, "g, seq_len_q, seq_len_k, head_dim_qk, head_dim_v must be positive");
  if (!q || !k || !v || !o) return fail(RB_INVALID_PARAM, "q, k, v and o must be device pointers");
  if (!(p->data_type == RB_F16 || p->data_type == RB_BF16))
    return fail(RB_UNSUPPORTED, "attention kernels exist for f16 and bf16");
  if (p->trans_q || p->trans_v || p->trans_o) return fail(RB_UNSUPPORTED, "transQ / transV / transO are not supported");
  if (p->head_qk % 64 || p->head_qk > 128 || p->head_v % 64 || p->head_v > 128)
    return fail(RB_UNSUPPORTED, "head dimensions must be 64 or 128");
  if (!p->trans_k && p->seq_k % 8) return fail(RB_UNSUPPORTED, "with K stored G x D x Sk, seq_len_k must be a multiple of 8");
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  AttMaps maps;
  memset(&maps, 0, sizeof(maps));
  const CUtensorMapDataType dt = p->data_type == RB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  std::string err;
  const uint64_t G = p->g, Sq = p->seq_q, Sk = p->seq_k, D = p->head_qk, Dv = p->head_v;
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
    const uint64_t str[2] = {Sk * 2, D * Sk * 2};
    const uint32_t box[3] = {64, (uint32_t)D, 1};
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
  kp.G = p->g; kp.Sq = p->seq_q; kp.Sk = p->seq_k; kp.D = p->head_qk; kp.Dv = p->head_v;
  kp.trans_k = p->trans_k ? 1 : 0;
  kp.is_bf16 = p->data_type == RB_BF16;
  kp.causal = p->causal ? 1 : 0;
  kp.q_tiles = (p->seq_q + kQT - 1) / kQT;
  kp.scale_log2 = (p->has_scale ? p->scale : 1.0f) * kLog2e;
  kp.bias = p->bias;
  kp.mask = p->mask;
  kp.mask_fill = p->mask_fill;
  const uint32_t fmt = kp.is_bf16 ? 1u : 0u;
  kp.idesc_s = make_idesc(1, fmt, fmt, 0, p->trans_k ? 0u : 1u, kQT, kKT);
  kp.idesc_pv = make_idesc(1, fmt, fmt, 0, 1u, kQT, (uint32_t)p->head_v);
  kp.status = dev->status_word;
  const long long ctas = (long long)p->g * kp.q_tiles;
  if (ctas > 0x7fffffffLL) return fail(RB_UNSUPPORTED, "too many query tiles");
  RB_CUDA_TRY(cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::kTotal));
  attention_fwd_kernel<<<(unsigned)ctas, kAttThreads, AttSmem::kTotal, stream>>>(maps, kp);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  return RB_SUCCESS;
}
