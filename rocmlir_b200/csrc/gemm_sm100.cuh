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
// The ring is walked in rounds of kpr K blocks (1, 2 or 4) that share one full / empty barrier pair: the barrier
// work of the single issuing threads is per round, and it is what bounds tiles whose MMAs are short.
// The epilogue has compact loops for the common cases (16-bit C, 4-byte C, fused elementwise work) beside a general
// one: the general body exceeds the instruction cache and runs an order of magnitude slower.
//
// Tile scheduler: static persistent loop with M-grouped rasterisation for L2 reuse, the same idea as
// rocMLIR's grouped grid layout (mlir/lib/Dialect/Rock/utility/GridLayoutEmitter.cpp:61-109).
#pragma once
#include "epilogue.cuh"
#include "ptx.cuh"

namespace rb {

constexpr int kBM = 128;          // rows of C per CTA
constexpr int kMaxBN = 256;       // widest tile: columns of C per tile (GemmParams::bn selects 64, 128 or 256)
constexpr int kRowBytes = 128;    // bytes of the contiguous dimension per shared-memory row (swizzle span)
constexpr int kGemmThreads = 256;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 8;        // M blocks per rasterisation group
#ifdef RB_ENABLE_PROBE
constexpr bool kProbeBuild = true;
#else
constexpr bool kProbeBuild = false;
#endif

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
  CUtensorMap c;  // store map of C (box: 128 bytes of a row x 32 rows); valid when GemmParams::c_tma != 0
};

// A operand fetched straight from an NHWC activation tensor (implicit GEMM): row m of A is output pixel m
// (n, p, q in row-major order), column (y, x, c) is in[n][p*stride + y*dil - pad][q*stride + x*dil - pad][c].
// One K block = one 128-byte run of channels of one filter tap.
// enabled == 2: the same for the B operand of a backward-weight convolution: K index = output pixel, column
// (y, x, c) = N index; one 64-element chunk of an MN-major B tile = one 128-byte run of channels of one tap.
struct ConvAParams {
  int enabled;
  int P, Q;             // output image
  int X;                // filter width (tap index = y * X + x)
  int cchunks;          // channel chunks (K blocks) per tap
  int stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
};

struct GemmParams {
  int G, M, N, K;
  int bn;                     // tile width in columns of C: UMMA N (a multiple of 32 * CTAS)
  int splits;                 // K is cut into `splits` ranges; with splits > 1 every range writes raw partial sums
  long long split_stride;     // elements between the partial planes of consecutive ranges (splits > 1)
  int tiles_m, tiles_n;       // tiles_m counts (kBM * CTAS)-row blocks
  int kblocks;                // K blocks per segment
  int nseg;
  uint32_t idesc;
  int acc_is_int;
  void* c;
  long long c_stride_g, c_stride_m, c_stride_n;  // in elements
  int c_type;
  int vec_ok;                 // rows of C start 16-byte aligned and c_stride_n == 1
  int c_tma;                  // C is written by TMA stores from a shared-memory staging tile
  EpiParams epi;
  uint32_t* status;
  unsigned long long* trace;  // optional [gridDim.x][16] cycle counters per CTA (see rbSetTraceBuffer), or NULL
  // Stream-K tail (only with splits == 1): the first dp_tiles tiles are computed whole, round-robin over the
  // persistent CTAs (pairs); the K blocks of the remaining sk_tiles tiles are dealt out evenly and contiguously,
  // so a CTA may compute only part of a tile's K range. The CTA that holds a tile's first K blocks owns the tile:
  // the others write f32/i32 partial tiles to sk_partial[unit] and raise sk_flags[unit]; the owner adds them in
  // unit order in its epilogue. Partial work comes first in every CTA's range and owned work last, so an owner
  // never waits for work that has not started.
  int dp_tiles, sk_tiles;
  void* sk_partial;            // [units][bn / 32][8][kBM * CTAS] 16-byte words of raw accumulators (row fastest: coalesced)
  unsigned int* sk_flags;      // [units][8]: one word per (CTA of the pair, epilogue warp), set to sk_token when written
  unsigned int sk_token;       // unique per launch, so stale words of earlier launches never match
  ConvAParams conva;
  int a_fused, b_fused;       // MN-major operand loaded with one 4-D box per stage (extent a multiple of the chunk)
  int probe;                  // instrumentation, only in builds with -DRB_ENABLE_PROBE (results become meaningless):
                              // bit0 = no loads, bit1 = no epilogue work, bit2 = epilogue without its global stores
  int stall;                  // failure-detection test hook (rbInjectStall): the producer issues no loads and never
                              // completes a stage, so every role's bounded wait runs out and the kernel returns with a
                              // status code instead of a result
  long long wait_cycles;      // budget of every bounded wait in SM cycles (rbSetWaitLimit; default kWaitCycles)
  int stages;                 // shared-memory ring depth (<= GemmSmemLayout::kMaxStages), a multiple of kpr
  int kpr;                    // K blocks per barrier round (1, 2 or 4): one full/empty barrier pair serves kpr ring slots
  // Channel-major convolution result (NKHW) written by the epilogue itself: row m = (image, pixel) with c_rows_per_img
  // pixels per image goes to image * c_img_stride + pixel * c_stride_m, column n adds n * c_stride_n. 0 = plain rows.
  int c_rows_per_img;
  long long c_img_stride;
  // Chained pair (G = 2, csrc/gemm_sm100.cu rbGemmGemm): group 1's A operand is group 0's result. The epilogue warps of a
  // group-0 tile raise chain_flags[m block][(n block, CTA, warp)] = chain_token once their rows are in global memory;
  // the producer of a group-1 tile waits for every word of its m block before its first load. Tiles are numbered group
  // 0 first and dealt round-robin, so a waiting CTA has finished all of its own group-0 tiles. chain_flip: bit 0 / 1 /
  // 2 = the tensor map of A / B / C holds group 1 at the lower address (group coordinate = g ^ 1).
  unsigned int* chain_flags;
  unsigned int chain_token;
  int chain_flip;
};

// Implicit B operand: base coordinates of output pixel `pix` (row-major n, p, q) and the tap / channel chunk of
// column `col`. Columns past the end of the matrix fetch tap 0 (their results are never stored).
__device__ __forceinline__ void convb_pixel(const ConvAParams& cv, int pix, int& img, int& base_h, int& base_w) {
  const int pq = cv.P * cv.Q;
  img = pix / pq;
  const int rem = pix - img * pq;
  const int op = rem / cv.Q;
  base_h = op * cv.stride_h - cv.pad_h;
  base_w = (rem - op * cv.Q) * cv.stride_w - cv.pad_w;
}
__device__ __forceinline__ void convb_tap(const ConvAParams& cv, int col, int ncols, int che, int& cc, int& fy, int& fx) {
  const int chunk = (col < ncols) ? col / che : 0;
  const int tap = chunk / cv.cchunks;
  cc = chunk - tap * cv.cchunks;
  fy = tap / cv.X;
  fx = tap - fy * cv.X;
}

template <int CTAS>
struct GemmSmemLayout {
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kMaxStages = 8;
  static constexpr int kSmemBudget = 232448;  // opt-in shared memory per CTA on sm_100
  static constexpr int stage_bytes(int bn) { return kABytes + (bn / CTAS) * kRowBytes; }
  // Epilogue staging: per epilogue warp two 32-row x 128-byte tiles (double buffered TMA stores).
  static constexpr int kStoreTileBytes = 32 * kRowBytes;
  static constexpr int kStagingBytes = 4 * 2 * kStoreTileBytes;
  // With per-column epilogue vectors the staging is single-buffered: the 16 KB saved keep the ring at six 32 KB
  // stages (three rounds of two K blocks) beside the vectors, which matters more than overlapping the stores.
  static constexpr int staging_bytes(bool epi_vec) { return epi_vec ? kStagingBytes / 2 : kStagingBytes; }
  static constexpr int kBarBytes = 512;
  // Per-column epilogue vectors of the current tile as f32, one private copy per epilogue warp (no cross-warp
  // barrier is needed that way): [4 warps][scale[kMaxBN], bias[kMaxBN]].
  static constexpr int kEpiVecBytes = 4 * 2 * kMaxBN * 4;
  static constexpr int total(int stages, int bn, bool epi_vec) {
    return stages * stage_bytes(bn) + staging_bytes(epi_vec) + (epi_vec ? kEpiVecBytes : 0) + kBarBytes + 1024;  // + alignment slack
  }
  static constexpr int max_stages(int bn, bool epi_vec) {
    int s = (kSmemBudget - staging_bytes(epi_vec) - (epi_vec ? kEpiVecBytes : 0) - kBarBytes - 1024) / stage_bytes(bn);
    return s > kMaxStages ? kMaxStages : s;
  }
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

// Work items of one persistent CTA (or CTA pair) `unit` out of `units`. All roles of a CTA walk the same sequence.
struct WorkItem {
  int tile;            // linear tile index (g, m block, n block)
  int split;           // uniform K split: index of the K range (0 otherwise)
  int kb_begin, kb_end;
  int kind;            // 0 whole result, 1 owner of a tile whose tail other units compute, 2 contributor
  int first_contrib, n_contrib;  // owner: units first_contrib .. first_contrib + n_contrib - 1 hold the rest
};
struct WorkIter {
  int unit, units, splits, kblocks, kb_per_split, dp_items, dp_tiles;
  int i;               // next data-parallel item
  long long cur, end;  // stream-K range of this unit in K blocks over the sk tiles
  long long q, r;      // every unit gets q blocks, the first r units one more
  __device__ WorkIter(const GemmParams& p, int unit_, int units_) {
    unit = unit_; units = units_; splits = p.splits; kblocks = p.kblocks;
    kb_per_split = (p.kblocks + p.splits - 1) / p.splits;
    dp_tiles = p.dp_tiles;
    dp_items = p.dp_tiles * p.splits;
    i = unit;
    const long long total = (long long)p.sk_tiles * p.kblocks;
    q = total / units; r = total % units;
    cur = unit * q + min((long long)unit, r);
    end = cur + q + (unit < r ? 1 : 0);
  }
  __device__ bool next(WorkItem& w) {
    if (i < dp_items) {
      w.tile = i / splits; w.split = i - w.tile * splits;
      w.kb_begin = w.split * kb_per_split; w.kb_end = min(kblocks, w.kb_begin + kb_per_split);
      w.kind = 0; w.first_contrib = 0; w.n_contrib = 0;
      i += units;
      return true;
    }
    if (cur >= end) return false;
    const int t = (int)(cur / kblocks);
    w.tile = dp_tiles + t; w.split = 0;
    w.kb_begin = (int)(cur - (long long)t * kblocks);
    w.kb_end = (int)min((long long)kblocks, w.kb_begin + (end - cur));
    cur += w.kb_end - w.kb_begin;
    w.first_contrib = 0; w.n_contrib = 0;
    if (w.kb_begin != 0) { w.kind = 2; return true; }
    if (w.kb_end == kblocks) { w.kind = 0; return true; }
    w.kind = 1;
    w.first_contrib = unit + 1;
    long long remaining = kblocks - w.kb_end;
    for (int u = unit + 1; remaining > 0 && u < units; ++u) { remaining -= q + (u < r ? 1 : 0); ++w.n_contrib; }
    return true;
  }
};

// ---- Fused epilogue loops kept OUT of the kernel body -------------------------------------------------------------
// The kernel's per-tile path is latency-critical for problems with a short K loop (a pointwise convolution runs 42
// tiles of four K blocks per CTA), and its speed follows the size of the code around it: with these loops inlined -
// never executed by such a problem - the C = 256 -> K = 64 pointwise layers lost 12 % (forward) and 6 % (backward data).
// They are therefore separate functions, called by the tiles that need them.
struct EpiStoreCtx {
  const CUtensorMap* cmap;   // store map of C
  uint8_t* staging;          // this warp's staging buffers
  uint32_t stg_bufs;         // 1 or 2
  uint32_t taddr;            // this warp's quarter of the accumulator buffer
  int col0;                  // first column of the tile
  int bn, N, M;
  int row0, gz, lane;
};

// 16-bit C from float accumulators with the common float tails: [round to mid] -> [x alpha] -> [+ bias[n], round to mid]
// -> [ReLU] -> convert; the operations and their order are those of epi_apply32. Returns the updated store count.
static __device__ __noinline__ uint32_t epi_fused16_tile(const EpiStoreCtx c, uint32_t flags, int mid_type, float alpha,
                                                         const float* vec_bias, int c_type, uint32_t nstores) {
  const bool f_mid = (flags & RB_EPI_ROUND_MID) != 0, f_alpha = (flags & RB_EPI_ALPHA) != 0;
  const bool f_bias = (flags & RB_EPI_BIAS) != 0, f_relu = (flags & RB_EPI_RELU) != 0;
  const int nsteps = c.bn / 64;
#pragma unroll 1
  for (int cp = 0; cp < nsteps; ++cp) {
    const int n0 = c.col0 + cp * 64;
    if (n0 >= c.N) break;  // warp-uniform
    uint32_t v[64];
    tmem_ld32(c.taddr + cp * 64, v);
    tmem_ld32(c.taddr + cp * 64 + 32, v + 32);
    uint8_t* stg = c.staging + (c.stg_bufs == 2 ? (nstores & 1u) : 0u) * (32 * kRowBytes);
    if (c.lane == 0 && nstores >= c.stg_bufs) {   // the store that last used this buffer has read it
      if (c.stg_bufs == 2) bulk_wait_read<1>(); else bulk_wait_read<0>();
    }
    __syncwarp();
    tmem_ld_wait();
    if (f_mid) {
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(round_to_type(__uint_as_float(v[j]), mid_type));
    }
    if (f_alpha) {
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(__fmul_rn(__uint_as_float(v[j]), alpha));
    }
    if (f_bias) {
      const float* bs = vec_bias + cp * 64;
#pragma unroll
      for (int j = 0; j < 64; j += 4) {
        const float4 b4 = *reinterpret_cast<const float4*>(bs + j);
        v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), b4.x));
        v[j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 1]), b4.y));
        v[j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 2]), b4.z));
        v[j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 3]), b4.w));
      }
      if (f_mid) {
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(round_to_type(__uint_as_float(v[j]), mid_type));
      }
    }
    if (f_relu) {
#pragma unroll
      for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.0f));
    }
    uint8_t* rowp = stg + c.lane * kRowBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(v[8 * i + 2 * j]), hi = __uint_as_float(v[8 * i + 2 * j + 1]);
        if (c_type == RB_F16) { __half2 t2 = __floats2half2_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
        else { __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
      }
      *reinterpret_cast<uint4*>(rowp + ((i ^ (c.lane & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
    }
    fence_proxy_async();
    __syncwarp();
    if (c.lane == 0 && c.row0 < c.M) {
      tma_store_3d(c.cmap, stg, n0, c.row0, c.gz);
      bulk_commit();
    }
    ++nstores;
  }
  return nstores;
}

// Quantised linear layer: i32 accumulator x scale[n] x 1 / output scale -> i8 (round half even, saturate, plus the
// output zero point). 32 columns are 32 bytes of a staging row; four groups make one 128-byte-wide store.
static __device__ __noinline__ uint32_t epi_requant8_tile(const EpiStoreCtx c, const float* vec_scale, float recip, int zp,
                                                          uint32_t nstores) {
  const int ngroups = c.bn / 32;
#pragma unroll 1
  for (int g = 0; g < ngroups; ++g) {
    const int n0 = c.col0 + g * 32;
    if (n0 >= c.N) break;  // warp-uniform
    uint32_t v[32];
    tmem_ld32(c.taddr + g * 32, v);
    const int sub = g & 3;
    uint8_t* stg = c.staging + (c.stg_bufs == 2 ? (nstores & 1u) : 0u) * (32 * kRowBytes);
    if (sub == 0) {
      if (c.lane == 0 && nstores >= c.stg_bufs) { if (c.stg_bufs == 2) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
      __syncwarp();
    }
    tmem_ld_wait();
    const float* cs = vec_scale + g * 32;
    uint32_t wd[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 s4 = *reinterpret_cast<const float4*>(cs + 4 * i);
      const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
      uint32_t b = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x = __fmul_rn(__fmul_rn(__int2float_rn((int)v[4 * i + k]), sc[k]), recip);
        b |= (uint32_t)(uint8_t)(int8_t)f32_to_i8_zp(x, zp) << (8 * k);
      }
      wd[i] = b;
    }
    *reinterpret_cast<uint4*>(stg + c.lane * kRowBytes + (((sub * 2) ^ (c.lane & 7)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    *reinterpret_cast<uint4*>(stg + c.lane * kRowBytes + (((sub * 2 + 1) ^ (c.lane & 7)) << 4)) = make_uint4(wd[4], wd[5], wd[6], wd[7]);
    const bool last_group = (sub == 3) || (n0 + 32 >= c.N) || (g == ngroups - 1);
    if (last_group) {
      fence_proxy_async();
      __syncwarp();
      if (c.lane == 0 && c.row0 < c.M) {
        tma_store_3d(c.cmap, stg, n0 - sub * 32, c.row0, c.gz);
        bulk_commit();
      }
      ++nstores;
    }
  }
  return nstores;
}


// EPI: the instantiation that carries the fused elementwise epilogues (RbEpilogue flags, C += A.B). Launches without
// one run the EPI = false instantiation, in which every such branch folds away: the per-tile path of problems with a
// short K loop follows the size of the code around it (measured: the pointwise C = 256 -> K = 64 layers lost 12 % and
// 6 % when two never-executed fused loops were added to the one kernel, inlined or not).
template <int KIND, bool A_MN, bool B_MN, int CTAS, bool EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmTensorMaps maps, const GemmParams p) {
  const uint32_t eflags = EPI ? p.epi.flags : 0u;   // compile-time zero without EPI
  using KT = KindTraits<KIND>;
  using L = GemmSmemLayout<CTAS>;
  constexpr int ES = KT::ES;
  constexpr int BKE = kRowBytes / ES;          // K elements per stage
  constexpr int CHE = kRowBytes / ES;          // MN elements per MN-major chunk
  constexpr int KSTEPS = BKE / KT::UMMA_K;     // MMAs per stage (always 4)
  constexpr int CHUNK_BYTES = BKE * kRowBytes; // one MN-major chunk: BKE k-rows of 128 B
  const int bn_cta = p.bn / CTAS;              // columns of B this CTA loads
  const int stage_bytes = L::stage_bytes(p.bn);
  const int probe = kProbeBuild ? p.probe : 0;  // folds to 0 (and every probe branch away) in the shipped build
  const long long wait_limit = p.wait_cycles;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  const int kpr = p.kpr;               // K blocks per barrier round
  const int rounds = stages / kpr;     // barrier pairs in use
  uint8_t* staging = smem + stages * stage_bytes;  // 1024-byte aligned (stage sizes are multiples of 1024)
  const bool epi_vec = epi_needs_col_vectors(eflags);
  float* epi_vecs = reinterpret_cast<float*>(staging + L::staging_bytes(epi_vec));   // present only when epi_vec
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + L::staging_bytes(epi_vec) + (epi_vec ? L::kEpiVecBytes : 0));
  uint64_t* full_bar = bars;                       // [stages]
  uint64_t* empty_bar = bars + stages;             // [stages]
  uint64_t* tfull_bar = bars + 2 * stages;         // [2]
  uint64_t* tempty_bar = bars + 2 * stages + 2;    // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * stages + 4);

  const int warp = threadIdx.x >> 5;
  const uint32_t rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const int pair_id = blockIdx.x / CTAS;
  const int num_pairs = gridDim.x / CTAS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
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
    if (p.c_tma) prefetch_tmap(&maps.c);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane_id() == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      long long w_empty = 0;
      WorkIter it(p, pair_id, num_pairs);
      WorkItem w;
      while (ok && it.next(w)) {
        int g, mb, nb;
        tile_coords(w.tile, p.tiles_m, p.tiles_n, g, mb, nb);
        const int m0 = (mb * CTAS + (int)rank) * kBM;
        const int n0 = nb * p.bn + (int)rank * bn_cta;
        const int kb_begin = w.kb_begin, kb_end = w.kb_end;
        const int ktotal = (kb_end - kb_begin) * p.nseg;
        const int ga = g ^ (p.chain_flip & 1), gb = g ^ ((p.chain_flip >> 1) & 1);
        if (p.chain_flags != nullptr && g == 1) {   // A of this tile is the result of group 0's tiles of the same m block
          const int nw = p.tiles_n * CTAS * 4;
          if (!flags_wait(p.chain_flags + (size_t)mb * nw, nw, p.chain_token, p.status, kStatusTimeoutAux + 2, wait_limit)) { ok = false; break; }
        }
        int img = 0, base_h = 0, base_w = 0;
        if (p.conva.enabled == 1) {
          const int pq = p.conva.P * p.conva.Q;
          img = m0 / pq;
          const int rem = m0 - img * pq;
          const int op = rem / p.conva.Q;
          base_h = op * p.conva.stride_h - p.conva.pad_h;
          base_w = (rem - op * p.conva.Q) * p.conva.stride_w - p.conva.pad_w;
        }
        int seg = 0, kb = kb_begin;
        // One barrier round covers up to kpr consecutive K blocks in ring slots s * kpr ... (s indexes rounds):
        // the barrier work of the issuing threads is per round, which is what bounds narrow tiles.
        for (int kk0 = 0; kk0 < ktotal; kk0 += kpr) {
          const int nblk = min(kpr, ktotal - kk0);
          const long long tw = p.trace ? clock64() : 0;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, p.status, kStatusTimeoutProducer + s, wait_limit)) { ok = false; break; }
          if (p.trace) w_empty += clock64() - tw;
          if (p.stall) {
            // injected stall: the stage is never filled
          } else if (probe & 1) {
            if (CTAS == 1 || rank == 0) mbar_arrive(&full_bar[s]);
          } else if constexpr (CTAS == 1) {
            mbar_expect_tx(&full_bar[s], nblk * stage_bytes);
          } else {
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * nblk * stage_bytes);
          }
          for (int j = 0; j < nblk; ++j) {
            uint8_t* sa = smem + (s * kpr + j) * stage_bytes;
            uint8_t* sb = sa + L::kABytes;
            const int k0 = kb * BKE;
            if ((probe & 1) || p.stall) {
              // loads switched off: the round's barrier was completed above (probe) or is left incomplete (stall)
            } else if constexpr (CTAS == 1) {
              if (!A_MN && p.conva.enabled == 1) {
                const int tap = kb / p.conva.cchunks, cc = kb - tap * p.conva.cchunks;
                const int fy = tap / p.conva.X, fx = tap - fy * p.conva.X;
                tma_load_im2col_4d(sa, &maps.a[seg], &full_bar[s], cc * BKE, base_w, base_h, img,
                                   (uint16_t)(fx * p.conva.dil_w), (uint16_t)(fy * p.conva.dil_h));
              } else if constexpr (!A_MN) {
                tma_load_3d(sa, &maps.a[seg], &full_bar[s], k0, m0, ga);
              } else if (p.a_fused) {
                tma_load_4d(sa, &maps.a[seg], &full_bar[s], 0, k0, m0 / CHE, ga);
              } else {
  #pragma unroll
                for (int c = 0; c < kBM / CHE; ++c)
                  tma_load_3d(sa + c * CHUNK_BYTES, &maps.a[seg], &full_bar[s], m0 + c * CHE, k0, ga);
              }
              if constexpr (!B_MN) {
                tma_load_3d(sb, &maps.b[seg], &full_bar[s], k0, n0, gb);
              } else if (p.conva.enabled == 2) {
                int bi, bh, bw;
                convb_pixel(p.conva, k0, bi, bh, bw);
                for (int c = 0; c < bn_cta / CHE; ++c) {
                  int cc, fy, fx;
                  convb_tap(p.conva, n0 + c * CHE, p.N, CHE, cc, fy, fx);
                  tma_load_im2col_4d(sb + c * CHUNK_BYTES, &maps.b[seg], &full_bar[s], cc * CHE, bw, bh, bi,
                                     (uint16_t)(fx * p.conva.dil_w), (uint16_t)(fy * p.conva.dil_h));
                }
              } else if (p.b_fused) {
                tma_load_4d(sb, &maps.b[seg], &full_bar[s], 0, k0, n0 / CHE, gb);
              } else {
                for (int c = 0; c < bn_cta / CHE; ++c)
                  tma_load_3d(sb + c * CHUNK_BYTES, &maps.b[seg], &full_bar[s], n0 + c * CHE, k0, gb);
              }
            } else {
              // Completion of this CTA's loads is counted on the leader CTA's barrier.
              const uint32_t lead_full = mapa_u32(smem_u32(&full_bar[s]), 0);
              if (!A_MN && p.conva.enabled == 1) {
                const int tap = kb / p.conva.cchunks, cc = kb - tap * p.conva.cchunks;
                const int fy = tap / p.conva.X, fx = tap - fy * p.conva.X;
                tma_load_im2col_4d_bar(sa, &maps.a[seg], lead_full, cc * BKE, base_w, base_h, img,
                                       (uint16_t)(fx * p.conva.dil_w), (uint16_t)(fy * p.conva.dil_h));
              } else if constexpr (!A_MN) {
                tma_load_3d_bar(sa, &maps.a[seg], lead_full, k0, m0, ga);
              } else if (p.a_fused) {
                tma_load_4d_bar(sa, &maps.a[seg], lead_full, 0, k0, m0 / CHE, ga);
              } else {
  #pragma unroll
                for (int c = 0; c < kBM / CHE; ++c)
                  tma_load_3d_bar(sa + c * CHUNK_BYTES, &maps.a[seg], lead_full, m0 + c * CHE, k0, ga);
              }
              if constexpr (!B_MN) {
                tma_load_3d_bar(sb, &maps.b[seg], lead_full, k0, n0, gb);
              } else if (p.conva.enabled == 2) {
                int bi, bh, bw;
                convb_pixel(p.conva, k0, bi, bh, bw);
                for (int c = 0; c < bn_cta / CHE; ++c) {
                  int cc, fy, fx;
                  convb_tap(p.conva, n0 + c * CHE, p.N, CHE, cc, fy, fx);
                  tma_load_im2col_4d_bar(sb + c * CHUNK_BYTES, &maps.b[seg], lead_full, cc * CHE, bw, bh, bi,
                                         (uint16_t)(fx * p.conva.dil_w), (uint16_t)(fy * p.conva.dil_h));
                }
              } else if (p.b_fused) {
                tma_load_4d_bar(sb, &maps.b[seg], lead_full, 0, k0, n0 / CHE, gb);
              } else {
                for (int c = 0; c < bn_cta / CHE; ++c)
                  tma_load_3d_bar(sb + c * CHUNK_BYTES, &maps.b[seg], lead_full, n0 + c * CHE, k0, gb);
              }
            }
            if (++kb == kb_end) { kb = kb_begin; ++seg; }
          }
          if (++s == (uint32_t)rounds) { s = 0; ph ^= 1u; }
        }
      }
      if (p.trace) p.trace[blockIdx.x * 16 + 1] = (unsigned long long)w_empty;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    // The tensor pipe accepts few MMAs ahead of the one it executes, so whatever the issuing thread does
    // between two MMAs is a bubble. The full-barrier test of the NEXT stage is therefore issued before
    // the MMAs of the current one and its result is consumed after them (its latency hides behind them).
    if (lane_id() == 0 && rank == 0) {
      uint32_t s = 0, ph = 0, t = 0;
      bool ok = true;
      long long w_full = 0, w_tempty = 0, t_kloop = 0;
      const long long t_begin = p.trace ? clock64() : 0;
      unsigned long long ns_begin = 0;
      if (p.trace) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_begin));
      bool ready = false;
      // Descriptor halves: constant high word; low word of stage 0, advanced by adds only.
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), A_MN ? CHUNK_BYTES : 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem) + L::kABytes, B_MN ? CHUNK_BYTES : 16);
      const uint32_t kStageStep = (uint32_t)stage_bytes >> 4;
      constexpr uint32_t kAStep = (A_MN ? KT::UMMA_K * kRowBytes : KT::UMMA_K * ES) >> 4;
      constexpr uint32_t kBStep = (B_MN ? KT::UMMA_K * kRowBytes : KT::UMMA_K * ES) >> 4;
      const uint32_t full0 = smem_u32(&full_bar[0]);
      const uint32_t empty0 = smem_u32(&empty_bar[0]);
      WorkIter it(p, pair_id, num_pairs);
      WorkItem w;
      for (; ok && it.next(w); ++t) {
        const uint32_t buf = t & 1u;
        const uint32_t bph = (t >> 1) & 1u;
        const long long tw0 = p.trace ? clock64() : 0;
        if (!mbar_wait(&tempty_bar[buf], bph ^ 1u, p.status, kStatusTimeoutMma + 0x10 + buf, wait_limit)) { ok = false; break; }
        if (p.trace) w_tempty += clock64() - tw0;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kMaxBN;
        uint32_t accum = 0;
        const int ktotal = (w.kb_end - w.kb_begin) * p.nseg;
        const long long tk0 = p.trace ? clock64() : 0;
        if (kpr == 1) {
          // one K block per round: the tight loop (at 256-column tiles the four MMAs of a block execute for 512
          // cycles and the loop below must issue them in less)
          for (int kk = 0; kk < ktotal; ++kk) {
            if (!ready) {
              const long long tw = p.trace ? clock64() : 0;
              if (!mbar_wait(&full_bar[s], ph, p.status, kStatusTimeoutMma + s, wait_limit)) { ok = false; break; }
              if (p.trace) w_full += clock64() - tw;
            }
            uint32_t ns = s + 1, nph = ph;
            if (ns == (uint32_t)stages) { ns = 0; nph ^= 1u; }
            const bool next_ready = mbar_test_wait_addr(full0 + ns * 8, nph);  // consumed after the MMAs below
            const uint32_t a_lo = a_lo0 + s * kStageStep;
            const uint32_t b_lo = b_lo0 + s * kStageStep;
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
              umma_ss<KIND, CTAS>(tmem_d, desc64(a_lo + k * kAStep, desc_hi), desc64(b_lo + k * kBStep, desc_hi), p.idesc,
                                  accum);
              accum = 1;
            }
            if constexpr (CTAS == 1) {
              tc_commit_addr1(empty0 + s * 8);
            } else {
              tc_commit_mask2(empty0 + s * 8, 3);
            }
            s = ns;
            ph = nph;
            ready = next_ready;
          }
        } else {
          for (int kk0 = 0; kk0 < ktotal; kk0 += kpr) {
            const int nblk = min(kpr, ktotal - kk0);
            if (!ready) {
              const long long tw = p.trace ? clock64() : 0;
              if (!mbar_wait(&full_bar[s], ph, p.status, kStatusTimeoutMma + s, wait_limit)) { ok = false; break; }
              if (p.trace) w_full += clock64() - tw;
            }
            // no tcgen05 fence here: the operands arrive through the async proxy (TMA) and are ordered by the
            // barrier itself; the fence after the accumulator-buffer wait above orders the TMEM accesses
            uint32_t ns = s + 1, nph = ph;
            if (ns == (uint32_t)rounds) { ns = 0; nph ^= 1u; }
            const bool next_ready = mbar_test_wait_addr(full0 + ns * 8, nph);  // consumed after the MMAs below
            uint32_t a_lo = a_lo0 + s * kpr * kStageStep;
            uint32_t b_lo = b_lo0 + s * kpr * kStageStep;
            for (int j = 0; j < nblk; ++j) {
  #pragma unroll
              for (int k = 0; k < KSTEPS; ++k) {
                umma_ss<KIND, CTAS>(tmem_d, desc64(a_lo + k * kAStep, desc_hi), desc64(b_lo + k * kBStep, desc_hi), p.idesc,
                                    accum);
                accum = 1;
              }
              a_lo += kStageStep;
              b_lo += kStageStep;
            }
            // Free the round's slots in every CTA of the pair once these MMAs have read them.
            if constexpr (CTAS == 1) {
              tc_commit_addr1(empty0 + s * 8);
            } else {
              tc_commit_mask2(empty0 + s * 8, 3);
            }
            s = ns;
            ph = nph;
            ready = next_ready;
          }
        }
        if (!ok) break;
        if (p.trace) t_kloop += clock64() - tk0;
        if constexpr (CTAS == 1) {
          tc_commit<1>(&tfull_bar[buf]);
        } else {
          tc_commit_mask2(smem_u32(&tfull_bar[buf]), 3);
        }
      }
      if (p.trace) {
        p.trace[blockIdx.x * 16 + 2] = (unsigned long long)w_full;
        p.trace[blockIdx.x * 16 + 3] = (unsigned long long)w_tempty;
        p.trace[blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - t_begin);  // MMA issue loop, total
        p.trace[blockIdx.x * 16 + 5] = t;
        p.trace[blockIdx.x * 16 + 8] = (unsigned long long)t_kloop;   // of the total: inside the K loops
        unsigned long long ns_end;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_end));
        p.trace[blockIdx.x * 16 + 15] = ns_end - ns_begin;  // the same loop in nanoseconds (gives the SM clock)
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    const int lane = lane_id();
    const int es_c = dtype_size(p.c_type);
    const int cols_per_store = kRowBytes / es_c;          // columns covered by one 128-byte staging row
    const int groups_per_store = cols_per_store / 32;     // 32-column TMEM loads per staging row: 1, 2 or 4
    const bool raw_i32 = p.acc_is_int && p.c_type == RB_I32 && eflags == 0;
    const uint32_t stg_bufs = epi_vec ? 1u : 2u;   // staging buffers per warp
    uint8_t* my_staging = staging + q * stg_bufs * L::kStoreTileBytes;
    uint32_t t = 0, nstores = 0;
    long long w_tfull = 0, e_work = 0, e_ld = 0, e_cv = 0;
    WorkIter it(p, pair_id, num_pairs);
    WorkItem w;
    for (; it.next(w); ++t) {
      int g, mb, nb;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, g, mb, nb);
      const uint32_t buf = t & 1u;
      const uint32_t bph = (t >> 1) & 1u;
      const long long tw = p.trace ? clock64() : 0;
      if (!mbar_wait_warp(&tfull_bar[buf], bph, p.status, kStatusTimeoutEpilogue + buf, wait_limit)) break;
      const long long te = p.trace ? clock64() : 0;
      w_tfull += te - tw;
      tc_fence_after();
      const long long row0 = (long long)(mb * CTAS + (int)rank) * kBM + q * 32;
      const long long row = row0 + lane;
      const bool row_ok = row < p.M;
      const int ngroups = p.bn / 32;
      const int gz = w.split * p.G + (g ^ ((p.chain_flip >> 2) & 1));   // group coordinate of the store map (K-split planes are stacked groups)
      // Per-column scales / biases of this tile, converted to f32, in this warp's private copy.
      float* vec_scale = epi_vecs + q * (2 * kMaxBN);
      float* vec_bias = vec_scale + kMaxBN;
      if (epi_vec) {
        __syncwarp();  // the previous tile's reads of the copy are done
        for (int j = lane; j < p.bn; j += 32) {
          const int n = min(nb * p.bn + j, p.N - 1);
          if (eflags & RB_EPI_COL_SCALE) vec_scale[j] = __ldg(p.epi.col_scale + n);
          if (epi_col_bias(eflags)) vec_bias[j] = load_bias(p.epi.bias, p.epi.bias_type, n);
        }
        __syncwarp();
      }
      long long c_row_off = (long long)w.split * p.split_stride + (long long)g * p.c_stride_g + row * p.c_stride_m;
      if (p.c_rows_per_img) {   // lanes of a warp are consecutive pixels: every column store covers 32 contiguous elements
        const long long img = row / p.c_rows_per_img;
        c_row_off = img * p.c_img_stride + (row - img * p.c_rows_per_img) * p.c_stride_m;
      }
      // what this thread's row contributes to the fused elementwise steps (row / scalar bias, residual address)
      EpiRow erow;
      if ((eflags & RB_EPI_BIAS) && (eflags & (RB_EPI_BIAS_ROW | RB_EPI_BIAS_SCALAR)))
        erow.row_bias = load_bias(p.epi.bias, p.epi.bias_type,
                                  (eflags & RB_EPI_BIAS_SCALAR) ? 0 : min(row, (long long)p.M - 1));
      erow.res_stride = p.c_stride_n;
      const int res_es = p.epi.res_type == RB_F32 ? 4 : 2;
      auto set_res = [&](int n0) {
        erow.ncols = min(32, p.N - n0);
        erow.res = (row_ok && (eflags & RB_EPI_RESIDUAL))
                       ? static_cast<const uint8_t*>(p.epi.residual) + (c_row_off + (long long)n0 * p.c_stride_n) * res_es
                       : nullptr;
      };
      // stream-K: 16-byte word i of column group c of this thread's row in the partial tile of unit u
      const int tile_row = (int)rank * kBM + q * 32 + lane;
      auto sk_word = [&](int u, int c, int i) -> uint4* {
        return reinterpret_cast<uint4*>(p.sk_partial) +
               (((size_t)u * ngroups + c) * 8 + i) * (size_t)(kBM * CTAS) + tile_row;
      };
      if (w.kind == 1) {
        // owner: the partial tiles it needs were produced at the start of the other units' ranges; this warp only
        // needs the rows written by the same warp of the same CTA of each contributing unit
        bool got = true;
        for (int u = w.first_contrib; u < w.first_contrib + w.n_contrib && got; ++u) {
          const volatile unsigned int* flag = p.sk_flags + u * 8 + (int)rank * 4 + q;
          const long long t0 = clock64();
          while (*flag != p.sk_token) {
            if (clock64() - t0 > wait_limit) { atomicCAS(p.status, 0u, kStatusTimeoutAux + 1); got = false; break; }
          }
        }
        __threadfence();
        if (!got) break;
      }
      // Fast path (whole tiles, float accumulators, no fused elementwise work, 16-bit C through TMA stores): a
      // compact loop - 64 columns = one 128-byte staging row per step. The general loop below handles every other
      // case; keeping this one small matters because the general loop's code is far larger than the instruction
      // cache and ran at about 1400 cycles per 32 columns where this one needs about 150.
      const bool fast16 = w.kind == 0 && p.c_tma && eflags == 0 && !p.acc_is_int && !probe &&
                          (p.c_type == RB_F16 || p.c_type == RB_BF16);
      // 4-byte C (f32 results, raw i32 results, the raw planes of a K split): 32 columns = one staging row per step
      const bool fast32 = w.kind == 0 && p.c_tma && !probe &&
                          ((eflags == 0 && !p.acc_is_int && p.c_type == RB_F32) || raw_i32);
      if (fast16) {
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN;
        const int nsteps = p.bn / 64;
#pragma unroll 1
        for (int cp = 0; cp < nsteps; ++cp) {
          const int n0 = nb * p.bn + cp * 64;
          if (n0 >= p.N) break;  // warp-uniform
          uint32_t v[64];
          tmem_ld32(taddr + cp * 64, v);
          tmem_ld32(taddr + cp * 64 + 32, v + 32);
          uint8_t* stg = my_staging + (nstores & 1u) * L::kStoreTileBytes;
          if (lane == 0 && nstores >= 2) bulk_wait_read<1>();  // the store that last used this buffer has read it
          __syncwarp();
          tmem_ld_wait();
          uint8_t* rowp = stg + lane * kRowBytes;
          if (p.c_type == RB_F16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              uint32_t h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __half2 t2 = __floats2half2_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                h[j] = *reinterpret_cast<uint32_t*>(&t2);
              }
              *reinterpret_cast<uint4*>(rowp + ((i ^ (lane & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              uint32_t h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                h[j] = *reinterpret_cast<uint32_t*>(&t2);
              }
              *reinterpret_cast<uint4*>(rowp + ((i ^ (lane & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && row0 < p.M) {
            tma_store_3d(&maps.c, stg, n0, (int)row0, gz);
            bulk_commit();
          }
          ++nstores;
        }
      } else if (fast32) {
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN;
#pragma unroll 1
        for (int c = 0; c < ngroups; ++c) {
          const int n0 = nb * p.bn + c * 32;
          if (n0 >= p.N) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          uint8_t* stg = my_staging + (nstores & 1u) * L::kStoreTileBytes;
          if (lane == 0 && nstores >= 2) bulk_wait_read<1>();
          __syncwarp();
          tmem_ld_wait();
          uint8_t* rowp = stg + lane * kRowBytes;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(rowp + ((i ^ (lane & 7)) << 4)) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && row0 < p.M) {
            tma_store_3d(&maps.c, stg, n0, (int)row0, gz);
            bulk_commit();
          }
          ++nstores;
        }
      }
      // The common float tails (per-tensor alpha, per-column bias, ReLU, roundings to a declared 16-bit type) and the
      // quantised linear layer have compact loops of their own, out of line (epi_fused16_tile, epi_requant8_tile).
      // Through the general loop GEMM + bias + ReLU took 31k cycles per tile, five times the plain store loop, and its
      // code evicted the other roles' instructions (the issue loop waited twice as long for operands).
      const bool f16_mid = (eflags & RB_EPI_ROUND_MID) && (p.epi.mid_type == RB_F16 || p.epi.mid_type == RB_BF16);
      const uint32_t f16_extra = eflags & ~(uint32_t)(RB_EPI_ALPHA | RB_EPI_BIAS | RB_EPI_RELU | (f16_mid ? RB_EPI_ROUND_MID : 0));
      const bool fast16e = eflags != 0 && w.kind == 0 && p.c_tma && f16_extra == 0 &&
                           (epi_col_bias(eflags) || !(eflags & RB_EPI_BIAS)) && !p.acc_is_int && !probe &&
                           (p.c_type == RB_F16 || p.c_type == RB_BF16);
      const bool fast8 = !fast16e && w.kind == 0 && p.c_tma && !probe && p.acc_is_int && p.c_type == RB_I8 &&
                         (eflags & ~(uint32_t)RB_EPI_ZP_OUT) == (uint32_t)(RB_EPI_COL_SCALE | RB_EPI_REQUANT);
      if (fast16e || fast8) {
        EpiStoreCtx ec;
        ec.cmap = &maps.c; ec.staging = my_staging; ec.stg_bufs = stg_bufs;
        ec.taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN;
        ec.col0 = nb * p.bn; ec.bn = p.bn; ec.N = p.N; ec.M = p.M; ec.row0 = (int)row0; ec.gz = gz; ec.lane = lane;
        if (fast16e) nstores = epi_fused16_tile(ec, eflags, p.epi.mid_type, p.epi.alpha, vec_bias, p.c_type, nstores);
        else nstores = epi_requant8_tile(ec, vec_scale, p.epi.out_recip, p.epi.out_zero, nstores);
      }
      // Channel-major f32 result of a convolution (NKHW): one store per column, the warp's 32 lanes are 32 consecutive
      // pixels of the column's image plane
      const bool fast_remap = w.kind == 0 && p.c_rows_per_img && eflags == 0 && !p.acc_is_int && !probe && p.c_type == RB_F32;
      if (fast_remap) {
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN;
#pragma unroll 1
        for (int c = 0; c < ngroups; ++c) {
          const int n0 = nb * p.bn + c * 32;
          if (n0 >= p.N) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
            float* d = static_cast<float*>(p.c) + c_row_off + (long long)n0 * p.c_stride_n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) d[(long long)j * p.c_stride_n] = __uint_as_float(v[j]);
          }
        }
      }
      // Fused elementwise work (or 1-byte / converted outputs) on whole tiles through TMA stores: the general loop's
      // body without its stream-K and plain-store branches.
      const bool fast_epi = !fast8 && !fast16 && !fast16e && !fast32 && !fast_remap && w.kind == 0 && p.c_tma && !probe && !raw_i32;
      if (fast_epi) {
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN;
#pragma unroll 1
        for (int c = 0; c < ngroups; ++c) {
          const int n0 = nb * p.bn + c * 32;
          if (n0 >= p.N) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          const int sub = c % groups_per_store;
          uint8_t* stg = my_staging + (stg_bufs == 2 ? (nstores & 1u) : 0u) * L::kStoreTileBytes;
          if (sub == 0) {
            if (lane == 0 && nstores >= stg_bufs) { if (stg_bufs == 2) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
            __syncwarp();
          }
          tmem_ld_wait();
          float x[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = p.acc_is_int ? __int2float_rn((int)v[j]) : __uint_as_float(v[j]);
          if (eflags) {
            set_res(n0);
            epi_apply32(x, p.epi, vec_scale + c * 32, vec_bias + c * 32, erow);
          }
          uint4 w4[8];
          const int nw = pack_row32(x, p.c_type, w4, p.epi.out_zero);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (i < nw) {
              const int piece = sub * nw + i;
              *reinterpret_cast<uint4*>(stg + lane * kRowBytes + ((piece ^ (lane & 7)) << 4)) = w4[i];
            }
          }
          const bool last_group = (sub == groups_per_store - 1) || (n0 + 32 >= p.N) || (c == ngroups - 1);
          if (last_group) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
              tma_store_3d(&maps.c, stg, n0 - sub * 32, (int)row0, gz);
              bulk_commit();
            }
            ++nstores;
          }
        }
      }
#pragma unroll 1
      for (int c = 0; c < ngroups && !fast8 && !fast16 && !fast16e && !fast32 && !fast_epi && !fast_remap; ++c) {
        const int n0 = nb * p.bn + c * 32;
        if (n0 >= p.N) break;  // warp-uniform
        if (probe & 2) break;
        uint32_t v[32];
        const long long tl0 = p.trace ? clock64() : 0;
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + buf * kMaxBN + c * 32, v);
        tmem_ld_wait();
        const long long tl1 = p.trace ? clock64() : 0;
        e_ld += tl1 - tl0;
        if (w.kind == 2) {  // contributor: raw accumulators to this unit's partial tile
#pragma unroll
          for (int i = 0; i < 8; ++i) *sk_word(pair_id, c, i) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          continue;
        }
        if (w.kind == 1) {  // owner: add the other units' partial tiles in unit order
          for (int u = w.first_contrib; u < w.first_contrib + w.n_contrib; ++u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint4 x4 = __ldcg(sk_word(u, c, i));
              if (p.acc_is_int) {
                v[4 * i] += x4.x; v[4 * i + 1] += x4.y; v[4 * i + 2] += x4.z; v[4 * i + 3] += x4.w;
              } else {
                v[4 * i] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * i]), __uint_as_float(x4.x)));
                v[4 * i + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * i + 1]), __uint_as_float(x4.y)));
                v[4 * i + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * i + 2]), __uint_as_float(x4.z)));
                v[4 * i + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * i + 3]), __uint_as_float(x4.w)));
              }
            }
          }
        }
        uint4 w4[8];
        int nw;
        if (raw_i32) {
#pragma unroll
          for (int i = 0; i < 8; ++i) w4[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          nw = 8;
        } else {
          float x[32];
          if (eflags == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = p.acc_is_int ? __int2float_rn((int)v[j]) : __uint_as_float(v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = p.acc_is_int ? __int2float_rn((int)v[j]) : __uint_as_float(v[j]);
            set_res(n0);
            epi_apply32(x, p.epi, vec_scale + c * 32, vec_bias + c * 32, erow);
          }
          if (p.c_tma || (p.vec_ok && n0 + 32 <= p.N)) {
            nw = pack_row32(x, p.c_type, w4, p.epi.out_zero);
          } else {
            nw = 0;
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) store_elem(p.c, c_row_off + (long long)(n0 + j) * p.c_stride_n, x[j], p.c_type, p.epi.out_zero);
            }
          }
        }
        if (p.trace) e_cv += clock64() - tl1;
        if (p.c_tma) {
          // Stage 32 rows x 128 bytes per store: row `lane` at lane * 128, its 16-byte pieces XOR-swizzled with
          // (lane & 7) exactly as the 128-byte-swizzled store map expects (also free of bank conflicts).
          const int sub = c % groups_per_store;
          uint8_t* stg = my_staging + (stg_bufs == 2 ? (nstores & 1u) : 0u) * L::kStoreTileBytes;
          if (sub == 0) {
            // the store that last used this buffer has read it
            if (lane == 0 && nstores >= stg_bufs) { if (stg_bufs == 2) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
            __syncwarp();
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (i < nw) {
              const int piece = sub * nw + i;
              *reinterpret_cast<uint4*>(stg + lane * kRowBytes + ((piece ^ (lane & 7)) << 4)) = w4[i];
            }
          }
          const bool last_group = (sub == groups_per_store - 1) || (n0 + 32 >= p.N) || (c == ngroups - 1);
          if (last_group) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row0 < p.M && !(probe & 4)) {
              tma_store_3d(&maps.c, stg, n0 - sub * 32, (int)row0, gz);
              bulk_commit();
            }
            ++nstores;
          }
        } else if (nw > 0 && row_ok && !(probe & 4)) {
          if (p.vec_ok && n0 + 32 <= p.N) {
            uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.c) + (c_row_off + n0) * es_c);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (i < nw) d[i] = w4[i];
          } else {  // raw i32 with a ragged or strided destination
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N)
                reinterpret_cast<int32_t*>(p.c)[c_row_off + (long long)(n0 + j) * p.c_stride_n] = (int32_t)v[j];
          }
        }
      }
      // This warp has drained its quarter of the accumulator buffer.
      tc_fence_before();
      __syncwarp();
      if (w.kind == 2) {
        __threadfence();          // the partial tile is visible before the flag
        __syncwarp();
        if (lane == 0) *reinterpret_cast<volatile unsigned int*>(p.sk_flags + pair_id * 8 + (int)rank * 4 + q) = p.sk_token;
      }
      if (lane == 0) {
        if constexpr (CTAS == 1) mbar_arrive(&tempty_bar[buf]);
        else mbar_arrive_cluster(&tempty_bar[buf], 0);
      }
      if (p.chain_flags != nullptr && g == 0) {
        // this warp's rows of the intermediate are complete in global memory before its flag says so
        if (p.c_tma && lane == 0) { bulk_wait<0>(); fence_proxy_async_all(); }
        __threadfence();
        __syncwarp();
        if (lane == 0)
          *reinterpret_cast<volatile unsigned int*>(p.chain_flags + (size_t)mb * (p.tiles_n * CTAS * 4) + (nb * CTAS + (int)rank) * 4 + q) = p.chain_token;
      }
      if (p.trace) e_work += clock64() - te;
    }
    if (p.c_tma && lane == 0) bulk_wait<0>();  // every store of this thread has completed before the CTA exits
    if (p.trace && warp == 4 && lane == 0) {
      p.trace[blockIdx.x * 16 + 6] = (unsigned long long)w_tfull;
      p.trace[blockIdx.x * 16 + 7] = (unsigned long long)e_work;
      p.trace[blockIdx.x * 16 + 13] = (unsigned long long)e_ld;   // of e_work: TMEM loads
      p.trace[blockIdx.x * 16 + 14] = (unsigned long long)e_cv;   //            conversion / fused elementwise / packing
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
