// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
// Replaces the main loop that rocMLIR generates for rock.gemm / implicit-GEMM rock.conv
// (GridwiseGemmAccelRewritePattern, mlir/lib/Dialect/Rock/Transforms/GridwiseGemmToBlockwise.cpp:2409-2811:
// global read -> LDS write -> MFMA, software-pipelined) with the Blackwell pipeline
//   TMA (plain, per-CTA loads) -> 128B-swizzled shared-memory ring -> tcgen05.mma -> TMEM accumulator
//   -> tcgen05.ld -> fused epilogue in registers -> global store.
//
// Roles inside one CTA (256 threads):
//   warp 0    producer: one lane issues the TMA loads of every stage
//   warp 1    MMA issuer: one lane issues tcgen05.mma and the commits that free stages / publish tiles
//   warp 2    TMEM allocator
//   warps 4-7 epilogue: warp (w & 3) owns TMEM lanes 32*(w & 3) .. +31, i.e. 32 rows of the tile
// Two TMEM accumulator buffers (2 x 256 columns) let the epilogue of tile i overlap the main loop of
// tile i+1. With CTAS == 2 two CTAs of a cluster form a pair that computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of A and its own 128 columns of B.
//
// Tile scheduler: static persistent loop with M-grouped rasterisation for L2 reuse, the same idea as
// rocMLIR's grouped grid layout (mlir/lib/Dialect/Rock/utility/GridLayoutEmitter.cpp:61-109).
#pragma once
#include "epilogue.cuh"
#include "ptx.cuh"

namespace rb {

constexpr int kBM = 128;          // rows of C per CTA
constexpr int kBN = 256;          // columns of C per tile
constexpr int kRowBytes = 128;    // bytes of the contiguous dimension per shared-memory row (swizzle span)
constexpr int kGemmThreads = 256;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 8;        // M blocks per rasterisation group

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<kKindF16> { static constexpr int ES = 2, UMMA_K = 16; };
template <>
struct KindTraits<kKindTF32> { static constexpr int ES = 4, UMMA_K = 8; };
template <>
struct KindTraits<kKindI8> { static constexpr int ES = 1, UMMA_K = 32; };
template <>
struct KindTraits<kKindF8> { static constexpr int ES = 1, UMMA_K = 32; };

// A contraction may be the sum of up to kMaxSeg (A_s, B_s) products over the same K range
// (3xTF32 split of an f32 GEMM). Segment s streams tiles from tensor maps tma[s] / tmb[s].
constexpr int kMaxSeg = 3;

struct GemmTensorMaps {
  CUtensorMap a[kMaxSeg];
  CUtensorMap b[kMaxSeg];
};

struct GemmParams {
  int G, M, N, K;
  int tiles_m, tiles_n;       // tiles_m counts (kBM * CTAS)-row blocks
  int kblocks;                // K blocks per segment
  int nseg;
  uint32_t idesc;
  int acc_is_int;
  void* c;
  long long c_stride_g, c_stride_m, c_stride_n;  // in elements
  int c_type;
  int vec_ok;                 // rows of C start 16-byte aligned and c_stride_n == 1
  EpiParams epi;
  uint32_t* status;
};

template <int CTAS>
struct GemmSmemLayout {
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = (kBN / CTAS) * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (CTAS == 1) ? 4 : 6;
  static constexpr int kBarBytes = 512;
  static constexpr int kTotal = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& g, int& mb, int& nb) {
  const int per_g = tiles_m * tiles_n;
  g = tile / per_g;
  int t = tile - g * per_g;
  const int per_group = kGroupM * tiles_n;
  const int grp = t / per_group;
  const int first_m = grp * kGroupM;
  const int gsz = min(kGroupM, tiles_m - first_m);
  t -= grp * per_group;
  mb = first_m + t % gsz;
  nb = t / gsz;
}

template <int KIND, bool A_MN, bool B_MN, int CTAS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmTensorMaps maps, const GemmParams p) {
  using KT = KindTraits<KIND>;
  using L = GemmSmemLayout<CTAS>;
  constexpr int ES = KT::ES;
  constexpr int BKE = kRowBytes / ES;          // K elements per stage
  constexpr int CHE = kRowBytes / ES;          // MN elements per MN-major chunk
  constexpr int KSTEPS = BKE / KT::UMMA_K;     // MMAs per stage (always 4)
  constexpr int BN_CTA = kBN / CTAS;           // columns of B this CTA loads
  constexpr int CHUNK_BYTES = BKE * kRowBytes; // one MN-major chunk: BKE k-rows of 128 B

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + L::kStages;         // [kStages]
  uint64_t* tfull_bar = bars + 2 * L::kStages;     // [2]
  uint64_t* tempty_bar = bars + 2 * L::kStages + 2;  // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * L::kStages + 4);

  const int warp = threadIdx.x >> 5;
  const uint32_t rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const int pair_id = blockIdx.x / CTAS;
  const int num_pairs = gridDim.x / CTAS;
  const int num_tiles = p.G * p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4 * CTAS);  // one arrival per epilogue warp of every CTA in the pair
    }
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<CTAS>(tmem_holder, kTmemCols);
    tmem_relinquish<CTAS>();
  }
  if (warp == 0 && lane_id() == 0) {
    for (int s = 0; s < p.nseg; ++s) {
      prefetch_tmap(&maps.a[s]);
      prefetch_tmap(&maps.b[s]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int ktotal = p.kblocks * p.nseg;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane_id() == 0) {
      uint32_t it = 0;
      bool ok = true;
      // Completion of this CTA's loads is counted on the leader CTA's barrier.
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        int g, mb, nb;
        tile_coords(tile, p.tiles_m, p.tiles_n, g, mb, nb);
        const int m0 = (mb * CTAS + (int)rank) * kBM;
        const int n0 = nb * kBN + (int)rank * BN_CTA;
        for (int kk = 0; kk < ktotal; ++kk, ++it) {
          const int seg = kk / p.kblocks;
          const int kb = kk - seg * p.kblocks;
          const uint32_t s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, p.status, kStatusTimeoutProducer + s)) { ok = false; break; }
          uint8_t* sa = smem + s * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const int k0 = kb * BKE;
          if constexpr (CTAS == 1) {
            mbar_expect_tx(&full_bar[s], L::kStageBytes);
            if constexpr (!A_MN) {
              tma_load_3d(sa, &maps.a[seg], &full_bar[s], k0, m0, g);
            } else {
#pragma unroll
              for (int c = 0; c < kBM / CHE; ++c)
                tma_load_3d(sa + c * CHUNK_BYTES, &maps.a[seg], &full_bar[s], m0 + c * CHE, k0, g);
            }
            if constexpr (!B_MN) {
              tma_load_3d(sb, &maps.b[seg], &full_bar[s], k0, n0, g);
            } else {
#pragma unroll
              for (int c = 0; c < BN_CTA / CHE; ++c)
                tma_load_3d(sb + c * CHUNK_BYTES, &maps.b[seg], &full_bar[s], n0 + c * CHE, k0, g);
            }
          } else {
            const uint32_t lead_full = mapa_u32(smem_u32(&full_bar[s]), 0);
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * L::kStageBytes);
            if constexpr (!A_MN) {
              tma_load_3d_bar(sa, &maps.a[seg], lead_full, k0, m0, g);
            } else {
#pragma unroll
              for (int c = 0; c < kBM / CHE; ++c)
                tma_load_3d_bar(sa + c * CHUNK_BYTES, &maps.a[seg], lead_full, m0 + c * CHE, k0, g);
            }
            if constexpr (!B_MN) {
              tma_load_3d_bar(sb, &maps.b[seg], lead_full, k0, n0, g);
            } else {
#pragma unroll
              for (int c = 0; c < BN_CTA / CHE; ++c)
                tma_load_3d_bar(sb + c * CHUNK_BYTES, &maps.b[seg], lead_full, n0 + c * CHE, k0, g);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane_id() == 0 && rank == 0) {
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++t) {
        const uint32_t buf = t & 1u;
        const uint32_t bph = (t >> 1) & 1u;
        if (!mbar_wait(&tempty_bar[buf], bph ^ 1u, p.status, kStatusTimeoutMma + 0x10 + buf)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kBN;
        for (int kk = 0; kk < ktotal; ++kk, ++it) {
          const uint32_t s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          if (!mbar_wait(&full_bar[s], ph, p.status, kStatusTimeoutMma + s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < KSTEPS; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * KT::UMMA_K * kRowBytes, CHUNK_BYTES, 1024)
                                        : make_smem_desc(sa + k * KT::UMMA_K * ES, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * KT::UMMA_K * kRowBytes, CHUNK_BYTES, 1024)
                                        : make_smem_desc(sb + k * KT::UMMA_K * ES, 16, 1024);
            umma_ss<KIND, CTAS>(tmem_d, adesc, bdesc, p.idesc, (kk | k) != 0 ? 1u : 0u);
          }
          // Free the stage in every CTA of the pair once these MMAs have read it.
          if constexpr (CTAS == 1) {
            tc_commit<1>(&empty_bar[s]);
          } else {
            tc_commit_addr2(mapa_u32(smem_u32(&empty_bar[s]), 0));
            tc_commit_addr2(mapa_u32(smem_u32(&empty_bar[s]), 1));
          }
        }
        if (!ok) break;
        if constexpr (CTAS == 1) {
          tc_commit<1>(&tfull_bar[buf]);
        } else {
          tc_commit_addr2(mapa_u32(smem_u32(&tfull_bar[buf]), 0));
          tc_commit_addr2(mapa_u32(smem_u32(&tfull_bar[buf]), 1));
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    const int lane = lane_id();
    uint32_t t = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++t) {
      int g, mb, nb;
      tile_coords(tile, p.tiles_m, p.tiles_n, g, mb, nb);
      const uint32_t buf = t & 1u;
      const uint32_t bph = (t >> 1) & 1u;
      if (!mbar_wait(&tfull_bar[buf], bph, p.status, kStatusTimeoutEpilogue + buf)) break;
      tc_fence_after();
      const long long row = (long long)(mb * CTAS + (int)rank) * kBM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int es_c = dtype_size(p.c_type);
      const long long c_row_off = (long long)g * p.c_stride_g + row * p.c_stride_m;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        const int n0 = nb * kBN + c * 32;
        if (n0 >= p.N) break;  // warp-uniform
        uint32_t v[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + buf * kBN + c * 32, v);
        tmem_ld_wait();
        const bool raw_i32 = p.acc_is_int && p.c_type == RB_I32 && p.epi.flags == 0;
        const bool full = (n0 + 32 <= p.N);
        if (raw_i32) {
          if (row_ok) {
            int32_t* dst = reinterpret_cast<int32_t*>(p.c);
            if (full && p.vec_ok) {
              uint4* d = reinterpret_cast<uint4*>(dst + c_row_off + n0);
#pragma unroll
              for (int i = 0; i < 8; ++i) d[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) dst[c_row_off + (long long)(n0 + j) * p.c_stride_n] = (int32_t)v[j];
            }
          }
        } else {
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float a = p.acc_is_int ? __int2float_rn((int)v[j]) : __uint_as_float(v[j]);
            const long long n = min((long long)(n0 + j), (long long)p.N - 1);
            x[j] = (p.epi.flags != 0) ? epi_apply(a, p.epi, n) : a;
          }
          if (row_ok) {
            if (full && p.vec_ok) {
              store_row32_vec(reinterpret_cast<uint8_t*>(p.c) + (c_row_off + n0) * es_c, x, p.c_type);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) store_elem(p.c, c_row_off + (long long)(n0 + j) * p.c_stride_n, x[j], p.c_type);
            }
          }
        }
      }
      // This warp has drained its quarter of the accumulator buffer.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 1) mbar_arrive(&tempty_bar[buf]);
        else mbar_arrive_cluster(&tempty_bar[buf], 0);
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, kTmemCols);
  }
}

}  // namespace rb
