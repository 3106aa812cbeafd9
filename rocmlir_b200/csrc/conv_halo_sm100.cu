// Unit-stride NHWC convolution (forward, and backward data as a forward convolution of the output gradient with
// mirrored taps) as an implicit GEMM that reads every input pixel from L2 ONCE per output tile.
//
// rocMLIR's implicit GEMM (ConvRewritePattern, mlir/lib/Dialect/Rock/Transforms/ConvToGemm.cpp:1133-1400) views the
// input through a pad -> embed -> merge coordinate map, so every filter tap re-reads its shifted window; the im2col-TMA
// form of this library (gemm_sm100.cuh) does the same and is bound by the L2 -> SM fabric for 3x3 filters (nine 16 KB
// tiles per 128 x 64 output tile). This kernel loads the tile's input window WITH ITS HALO once per 64-channel block:
//
//   * an output tile is R whole output rows of one image, indexed on the padded raster m = r * Wp + q with
//     Wp = Q + (X - 1) * dil_w (the columns q >= Q of a row are computed and thrown away); R * Wp <= 128;
//   * one TMA tiled load of the box {64 channels, Wp, R + (Y - 1) * dil_h, 1} starting at (w, h) = (-pad_w, p0 - pad_h)
//     puts the window into shared memory as [rows][Wp] pixels of 128 bytes, zero outside the image (the padding);
//   * on that raster the A operand of tap (y, x) is the SAME buffer shifted by y * dil_h * Wp + x * dil_w pixel rows:
//     a K-major 128-byte-swizzled tile whose start address is not on a 1024-byte boundary. The tensor core applies the
//     swizzle to absolute shared-memory address bits, exactly as the TMA engine did when it wrote the window, so the
//     shifted start address alone is enough: the descriptor's base-offset field stays 0 (measured on B200: results
//     are exact that way, and wrong when the field is set to the start's row phase);
//   * the filter matrix B[k][(y, x, c)] stays resident in shared memory for all tiles of the persistent CTA.
// Per tile the tensor pipe sees the same Y * X * C / 16 MMAs as before, but L2 -> SM traffic drops from
// Y * X * (16 + N / 8) KB to about (R + Y - 1) * Wp / 8 KB per channel block.
//
// Roles, barriers, TMEM double buffering and bounded waits are those of gemm_tcgen05_kernel.
#include <cuda_runtime.h>

#include <algorithm>
#include <string>

#include "epilogue.cuh"
#include "lib_state.h"
#include "ptx.cuh"

namespace rb {
namespace {

constexpr int kHaloThreads = 384;   // producer, MMA, TMEM and one idle warp, then two epilogue groups of four warps
constexpr int kHaloMaxStages = 6;
constexpr int kHaloMaxTaps = 49;   // up to 7 x 7 filters

struct HaloMaps {
  CUtensorMap in;    // {C, W, H, N} of the NHWC image tensor, box {64, Wp, rows_box, 1}
  CUtensorMap fil;   // {Y * X * C, Kout, 1} of the K-major filter matrix, box {64, Kout, 1}; or, for a filter read as it
                     // lies (b_mn), {Kout, FX, FY, Kfil} of the KYXC filter tensor, box {64, 1, 1, 64}
};

struct HaloParams {
  int N, P, Q, Kout, cchunks;       // output image P x Q with Kout channels; input channels = cchunks * 64
  int Y, X, dil_h, dil_w, pad_h, pad_w;
  int Wp, R, rows_box;              // padded raster width, output rows per 128-row sub-tile, input rows per box
  int G;                            // sub-tiles per stage: one window of G * R output rows feeds G accumulators (G * Kout <= 256)
  int slack_bytes;                  // rows past the last stage that shifted descriptors may touch
  int tiles_per_img, num_tiles;
  int stage_bytes, stages;
  int b_tile_bytes, b_tiles;        // one (tap, channel block) slab of the filter: Kout rows of 128 bytes
  int b_mn;                         // backward data from the KYXC filter itself: the slab is MN-major (64 rows of the
                                    // reduction index k, each 64 contiguous input channels; Kout / 64 such chunks)
  int fy0, fsy, fx0, fsx;           //   filter tap of raster tap (y', x') = (fy0 + fsy * (Y-1-y'), fx0 + fsx * (X-1-x'))
  uint32_t idesc;
  int is_bf16;
  void* out;                        // output pixels of Kout contiguous channels
  long long o_n, o_p, o_q;          // element strides of the output pixel (n, p, q)
  EpiParams epi;                    // fused elementwise tail over the output channel (flags == 0: none)
  int out_type;                     // RbDType of `out` when the epilogue converts (else the 16-bit element type)
  int wide_store;                   // `out` is 32-byte aligned: the plain epilogue stores 32 bytes at a time
  uint32_t* status;
  long long wait_cycles;
  unsigned long long* trace;        // optional [gridDim.x][16] cycle counters (rbSetTraceBuffer): [2] MMA thread waited for
                                    // a window, [3] for an accumulator, [4] its loop in total, [5] tiles, [6] epilogue
                                    // waited for a tile, [7] epilogue busy
};

// Up to four convolutions of one launch (the stride classes of a strided backward-data convolution): CTAs
// [first_cta[i], first_cta[i + 1]) work on convolution i with its own tensor maps, tile raster and resident filter.
constexpr int kHaloMaxGroup = 4;
struct HaloGroup {
  HaloMaps maps[kHaloMaxGroup];
  HaloParams prm[kHaloMaxGroup];
  int first_cta[kHaloMaxGroup + 1];
  int n;
};

// EPI = false is the plain store of the 16-bit result; the fused elementwise tail lives in its own instantiation so that
// its (large) code does not share the instruction cache with the plain kernel's loops.
template <bool EPI>
__global__ void __launch_bounds__(kHaloThreads, 1)
conv_halo_kernel(const __grid_constant__ HaloGroup g) {
  int member = 0;
#pragma unroll
  for (int i = 1; i < kHaloMaxGroup; ++i)
    if (i < g.n && (int)blockIdx.x >= g.first_cta[i]) member = i;
  const HaloParams& p = g.prm[member];
  const HaloMaps& maps = g.maps[member];
  const int cta = (int)blockIdx.x - g.first_cta[member], ctas = g.first_cta[member + 1] - g.first_cta[member];
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [A ring: stages * stage_bytes][slack: rows that shifted descriptors may touch past the last stage][B][barriers]
  uint8_t* b_smem = smem + p.stages * p.stage_bytes + p.slack_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_smem + p.b_tiles * p.b_tile_bytes);
  uint64_t* full_bar = bars;                      // [stages]
  uint64_t* empty_bar = bars + kHaloMaxStages;    // [stages]
  uint64_t* tfull_bar = bars + 2 * kHaloMaxStages;       // [2]
  uint64_t* tempty_bar = bars + 2 * kHaloMaxStages + 2;  // [2]
  uint64_t* bfull_bar = bars + 2 * kHaloMaxStages + 4;   // [1]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kHaloMaxStages + 5);
  const int warp = warp_id_uniform();
  const long long wait_limit = p.wait_cycles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
    mbar_init(bfull_bar, 1);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<1>(tmem_holder, 512);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane_id() == 0) { prefetch_tmap(&maps.in); prefetch_tmap(&maps.fil); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane_id() == 0) {
      // the filter, once: slab (tap, cc) = Kout rows x 64 channels
      mbar_expect_tx(bfull_bar, (uint32_t)(p.b_tiles * p.b_tile_bytes));
      if (!p.b_mn) {
        for (int j = 0; j < p.b_tiles; ++j) tma_load_3d(b_smem + (size_t)j * p.b_tile_bytes, &maps.fil, bfull_bar, j * 64, 0, 0);
      } else {
        // mirrored taps straight from the filter tensor: no rearranged copy of the filter exists
        for (int j = 0; j < p.b_tiles; ++j) {
          const int tap = j / p.cchunks, cc = j - tap * p.cchunks;
          const int ty = tap / p.X, tx = tap - ty * p.X;
          const int fy = p.fy0 + p.fsy * (p.Y - 1 - ty), fx = p.fx0 + p.fsx * (p.X - 1 - tx);
          for (int nc = 0; nc < p.Kout / 64; ++nc)
            tma_load_4d(b_smem + (size_t)j * p.b_tile_bytes + (size_t)nc * 8192, &maps.fil, bfull_bar, nc * 64, fx, fy, cc * 64);
        }
      }
      uint32_t s = 0, ph = 0;
      bool ok = true;
      const uint32_t box_bytes = (uint32_t)(p.Wp * p.rows_box * 128);
      for (int tile = cta; ok && tile < p.num_tiles; tile += ctas) {
        const int n = tile / p.tiles_per_img;
        const int p0 = (tile - n * p.tiles_per_img) * p.R * p.G;
        for (int cc = 0; cc < p.cchunks; ++cc) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, p.status, kStatusTimeoutProducer + s, wait_limit)) { ok = false; break; }
          mbar_expect_tx(&full_bar[s], box_bytes);
          tma_load_4d(smem + (size_t)s * p.stage_bytes, &maps.in, &full_bar[s], cc * 64, -p.pad_w, p0 - p.pad_h, n);
          if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the loop (so that its counters and descriptor addresses are warp-uniform values) and one elected
    // lane issues the tensor-core instructions and their commits.
    // one lane, chosen once: the commits must come from the thread that issued the MMAs they track
    const bool leader = elect_one();
    // the loop's invariants, read once (the parameter block is indexed by the group member)
    const int Y = p.Y, X = p.X, cchunks = p.cchunks, num_tiles = p.num_tiles, G = p.G, Kout = p.Kout;
    const uint32_t g_step = (uint32_t)(p.R * p.Wp) * 8u;   // one sub-tile down the window, in 16-byte units
    const uint32_t stages = (uint32_t)p.stages, idesc = p.idesc;
    const bool tracing = p.trace != nullptr;
    uint32_t* const status = p.status;
    bool ok = mbar_wait_warp(bfull_bar, 0, status, kStatusTimeoutMma + 0x20, wait_limit);
    uint32_t s = 0, ph = 0, t = 0;
    bool ready = false, tready = false;
    const uint32_t desc_hi0 = smem_desc_hi(1024);
    // descriptor-address steps in 16-byte units: one tap to the right, one tap row down, one filter slab on
    const uint32_t a_xstep = (uint32_t)p.dil_w * 8u, a_ystep = (uint32_t)(p.dil_h * p.Wp) * 8u;
    const uint32_t b_slab = (uint32_t)p.b_tile_bytes >> 4, b_tapstep = b_slab * (uint32_t)cchunks;
    long long w_full = 0, w_tempty = 0;
    const long long t_begin = tracing ? clock64() : 0;
    const uint32_t b_lo0 = smem_desc_lo(smem_u32(b_smem), p.b_mn ? 8192u : 16u);   // MN-major: 8 KB between 64-channel chunks
    const uint32_t b_kstep = p.b_mn ? 128u : 2u;   // one K step of 16: sixteen 128-byte rows, or 32 bytes along the row
    const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), 16);
    const uint32_t a_stage = (uint32_t)p.stage_bytes >> 4;
    for (int tile = cta; ok && tile < num_tiles; tile += ctas, ++t) {
      const uint32_t buf = t & 1u, bph = (t >> 1) & 1u;
      if (!tready) {
        const long long tw0 = tracing ? clock64() : 0;
        if (!mbar_wait_warp(&tempty_bar[buf], bph ^ 1u, status, kStatusTimeoutMma + 0x10 + buf, wait_limit)) { ok = false; break; }
        if (tracing) w_tempty += clock64() - tw0;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * 256;
      for (int cc = 0; cc < cchunks && ok; ++cc) {
        if (!ready) {
          const long long tw = tracing ? clock64() : 0;
          if (!mbar_wait_warp(&full_bar[s], ph, status, kStatusTimeoutMma + s, wait_limit)) { ok = false; break; }
          if (tracing) w_full += clock64() - tw;
          tc_fence_after();
        }
        // the NEXT stage's barrier, and after the last channel chunk the next tile's accumulator, are tested just
        // before this stage's last tap is issued, so that the answers arrive while those MMAs queue up
        uint32_t ns = s + 1, nph = ph;
        if (ns == stages) { ns = 0; nph ^= 1u; }
        bool next_ready = false, next_tready = false;
        const bool last_cc = cc + 1 == cchunks;
        // every tap is the same window, shifted: the swizzle pattern follows the absolute address, so the shifted
        // start address is all the descriptor needs
        for (int gsub = 0; gsub < G; ++gsub) {
        uint32_t a_row = a_lo0 + s * a_stage + (uint32_t)gsub * g_step;
        uint32_t b_lo = b_lo0 + (uint32_t)cc * b_slab;
        const uint32_t tmem_dg = tmem_d + (uint32_t)(gsub * Kout);
        uint32_t accum = cc ? 1u : 0u;
        for (int y = 0; y < Y; ++y) {
          uint32_t a_lo = a_row;
          for (int x = 0; x < X; ++x) {
            if (gsub + 1 == G && y + 1 == Y && x + 1 == X) {
              uint32_t f = mbar_test_wait(&full_bar[ns], nph) ? 1u : 0u;
              if (last_cc && mbar_test_wait(&tempty_bar[buf ^ 1u], (((t + 1) >> 1) & 1u) ^ 1u)) f |= 2u;
              f = __shfl_sync(0xffffffffu, f, 0);
              next_ready = f & 1u;
              next_tready = f & 2u;
            }
            if (leader) {
#pragma unroll
              for (int k = 0; k < 4; ++k)   // 64 channels = four K steps of 16
                umma_ss<kKindF16, 1>(tmem_dg, desc64(a_lo + k * 2, desc_hi0), desc64(b_lo + k * b_kstep, desc_hi0), idesc, k ? 1u : accum);
            }
            accum = 1;
            a_lo += a_xstep;
            b_lo += b_tapstep;
          }
          a_row += a_ystep;
        }
        }
        if (leader) tc_commit_addr1(smem_u32(&empty_bar[s]));
        s = ns; ph = nph; ready = next_ready;
        if (last_cc) tready = next_tready;
      }
      if (!ok) break;
      if (leader) tc_commit<1>(&tfull_bar[buf]);
    }
    if (tracing && lane_id() == 0) {
      p.trace[blockIdx.x * 16 + 2] = (unsigned long long)w_full;
      p.trace[blockIdx.x * 16 + 3] = (unsigned long long)w_tempty;
      p.trace[blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - t_begin);
      p.trace[blockIdx.x * 16 + 5] = t;
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ------------------------------
    const int q4 = warp & 3, lane = lane_id();
    const int m = q4 * 32 + lane;              // position on the tile's padded raster
    const int Wp = p.Wp, R = p.R, P = p.P, Q = p.Q, Kout = p.Kout, tiles_per_img = p.tiles_per_img, num_tiles = p.num_tiles, G = p.G;
    const long long o_n = p.o_n, o_p = p.o_p, o_q = p.o_q;
    const bool is_bf16 = p.is_bf16 != 0, wide = p.wide_store != 0, tracing = p.trace != nullptr;
    uint8_t* const out = static_cast<uint8_t*>(p.out);
    const int rr = m / Wp, qq = m - rr * Wp;
    uint32_t t = 0;
    long long w_tfull = 0, e_work = 0;
    // Two epilogue groups (warps 4-7 and 8-11): each serves one of the two accumulator buffers, i.e. every other tile,
    // so that layers whose tiles have little reduction work per output (few taps, many output channels) are not bound
    // by one group's drain rate.
    const uint32_t egroup = (uint32_t)(warp - 4) >> 2;
    for (int tile = cta; tile < num_tiles; tile += ctas, ++t) {
      const uint32_t buf = t & 1u, bph = (t >> 1) & 1u;
      if (buf != egroup) continue;
      const long long tw = tracing ? clock64() : 0;
      if (!mbar_wait_warp(&tfull_bar[buf], bph, p.status, kStatusTimeoutEpilogue + buf, wait_limit)) break;
      const long long te = tracing ? clock64() : 0;
      w_tfull += te - tw;
      tc_fence_after();
      const int n = tile / tiles_per_img;
      for (int gsub = 0; gsub < G; ++gsub) {
      const int p0 = (tile - n * tiles_per_img) * R * G + gsub * R;
      const bool valid = rr < R && qq < Q && p0 + rr < P;
      const long long pix = (long long)n * o_n + (long long)(p0 + rr) * o_p + (long long)qq * o_q;   // elements
      const uint32_t taddr = tmem_base + (uint32_t(q4 * 32) << 16) + buf * 256 + (uint32_t)(gsub * Kout);
      if constexpr (!EPI) {
        uint8_t* dst = out + 2 * pix;
#pragma unroll 1
        for (int c = 0; c < Kout; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          tmem_ld_wait();
          uint32_t h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float lo = __uint_as_float(v[2 * j]), hi = __uint_as_float(v[2 * j + 1]);
            if (is_bf16) { __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
            else { __half2 t2 = __floats2half2_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
          }
          if (valid) {
            if (wide) {   // 32 bytes per store: half as many trips through the load/store unit
              st_global_v8(dst + c * 2, h);
              st_global_v8(dst + c * 2 + 32, h + 8);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(dst + c * 2 + i * 16) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
            }
          }
        }
      } else {
        // fused tail (bias / scale per output channel, residual, relu, clip, requantisation): the same steps in the
        // same order as the GEMM kernel's epilogue; the per-channel vectors are read through the read-only cache
        const int es_o = dtype_size(p.out_type);
        uint8_t* dst = out + (long long)es_o * pix;
        EpiRow erow;
        if ((p.epi.flags & RB_EPI_BIAS) && (p.epi.flags & RB_EPI_BIAS_SCALAR)) erow.row_bias = load_bias(p.epi.bias, p.epi.bias_type, 0);
        erow.res_stride = 1;
        erow.ncols = 32;
#pragma unroll 1
        for (int c = 0; c < Kout; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          tmem_ld_wait();
          float xv[32], cs[32], bs[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            xv[j] = __uint_as_float(v[j]);
            cs[j] = (p.epi.flags & RB_EPI_COL_SCALE) ? __ldg(p.epi.col_scale + c + j) : 1.0f;
            bs[j] = epi_col_bias(p.epi.flags) ? load_bias(p.epi.bias, p.epi.bias_type, c + j) : 0.0f;
          }
          erow.res = (valid && (p.epi.flags & RB_EPI_RESIDUAL))
                         ? static_cast<const uint8_t*>(p.epi.residual) + (p.epi.res_type == RB_F32 ? 4 : 2) * (pix + c)
                         : nullptr;
          epi_apply32(xv, p.epi, cs, bs, erow);
          uint4 w4[8];
          const int nw = pack_row32(xv, p.out_type, w4, p.epi.out_zero);
          if (valid) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (i < nw) *reinterpret_cast<uint4*>(dst + c * es_o + i * 16) = w4[i];
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (tracing) e_work += clock64() - te;
    }
    if (tracing && warp == 4 && lane == 0) {   // group 0 only: its waits and work cover every other tile
      p.trace[blockIdx.x * 16 + 6] = (unsigned long long)w_tfull;
      p.trace[blockIdx.x * 16 + 7] = (unsigned long long)e_work;
    }
  }
  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

}  // namespace

bool conv_halo_applicable(const HaloConv& c) {
  if (c.C % 64 || c.Kout % 32 || c.Kout > 256 || c.Kout < 32) return false;
  if (c.b_mn && (c.Kout % 64 || (c.f_sk * 2) % 16 || (c.f_sy * 2) % 16 || (c.f_sx * 2) % 16)) return false;
  if (c.dil_h < 1 || c.dil_w < 1 || c.pad_h < 0 || c.pad_w < 0 || c.Y * c.X > 49) return false;
  const int Wp = c.Q + (c.X - 1) * c.dil_w;
  if (Wp > 128 || Wp != c.W + c.pad_w + c.pad_w_r) return false;
  if (c.P + (c.Y - 1) * c.dil_h != c.H + c.pad_h + c.pad_h_r) return false;
  const int R = std::min(128 / Wp, c.P);
  const int rows_box = R + (c.Y - 1) * c.dil_h;
  if (R < 1 || rows_box > 256 || Wp > 256) return false;
  const long long b_bytes = (long long)c.Y * c.X * (c.C / 64) * c.Kout * 128;
  const int stage_bytes = (Wp * rows_box + 7) / 8 * 8 * 128;
  // the filter stays resident beside at least two stages of the window ring
  const long long slack = ((128 - R * Wp + (c.X - 1) * c.dil_w + 7) / 8 * 8 + 8) * 128;
  return b_bytes + 2LL * stage_bytes + slack + 2048 <= 232448 - 1024;
}

namespace {

// Fills the kernel's description of one convolution; `smem` returns the dynamic shared memory it wants.
RbStatus halo_setup(const HaloConv& c, const void* image, const void* filter_matrix, void* out, const RbEpilogue* epi,
                    int out_type, const DeviceInfo* dev, HaloParams& p, HaloMaps& maps, int* smem) {
  if (!conv_halo_applicable(c)) return fail(RB_UNSUPPORTED, "convolution outside the reach of the halo kernel");
  memset(&p, 0, sizeof(p));
  p.N = c.N; p.P = c.P; p.Q = c.Q; p.Kout = c.Kout; p.cchunks = c.C / 64;
  p.Y = c.Y; p.X = c.X; p.dil_h = c.dil_h; p.dil_w = c.dil_w; p.pad_h = c.pad_h; p.pad_w = c.pad_w;
  p.Wp = c.Q + (c.X - 1) * c.dil_w;
  p.R = std::min(128 / p.Wp, c.P);
  p.b_tile_bytes = c.Kout * 128;
  p.b_tiles = c.Y * c.X * p.cchunks;
  if (c.Y * c.X > kHaloMaxTaps) return fail(RB_UNSUPPORTED, "halo kernel: filter larger than 7 x 7");
  // a shifted 128-row view of the last sub-tile may run past the window by the raster's unused rows plus the widest
  // horizontal tap offset: that many rows (rounded up to the swizzle atom) stay free behind the ring
  p.slack_bytes = ((128 - p.R * p.Wp + (c.X - 1) * c.dil_w + 7) / 8 * 8 + 8) * 128;
  int fixed = 0;
  // Two sub-tiles per stage when two accumulators fit a TMEM buffer and three stages still fit beside the filter:
  // one window of 2 R output rows shares its halo rows and halves the barrier work per output row.
  // (measured at C4a: one sub-tile 783, two 825, three 788, four 819 TFLOP/s on the same box)
  for (p.G = 2; p.G >= 1; --p.G) {
    if (p.G > 1 && (p.G * c.Kout > 256 || c.P <= (p.G - 1) * p.R)) continue;
    p.rows_box = p.G * p.R + (c.Y - 1) * c.dil_h;
    p.stage_bytes = (p.Wp * p.rows_box + 7) / 8 * 8 * 128;
    fixed = p.slack_bytes + p.b_tiles * p.b_tile_bytes + 2048;
    p.stages = std::min(kHaloMaxStages, (232448 - 1024 - fixed) / p.stage_bytes);
    if (p.rows_box <= 256 && p.stages >= (p.G == 2 ? 3 : 2)) break;
  }
  if (p.G < 1) return fail(RB_UNSUPPORTED, "halo kernel: the filter leaves no room for the window ring");
  p.tiles_per_img = (c.P + p.G * p.R - 1) / (p.G * p.R);
  p.num_tiles = c.N * p.tiles_per_img;
  const uint32_t fmt = c.is_bf16 ? 1u : 0u;
  p.idesc = make_idesc(1, fmt, fmt, 0, c.b_mn ? 1u : 0u, 128, (uint32_t)c.Kout);
  p.b_mn = c.b_mn ? 1 : 0;
  p.fy0 = c.fy0; p.fsy = c.fsy; p.fx0 = c.fx0; p.fsx = c.fsx;
  p.is_bf16 = c.is_bf16;
  p.out = out;
  p.o_n = c.o_n; p.o_p = c.o_p; p.o_q = c.o_q;
  p.out_type = out_type >= 0 ? out_type : (c.is_bf16 ? RB_BF16 : RB_F16);
  if (epi && epi->flags) {
    p.epi.flags = epi->flags; p.epi.alpha = epi->alpha; p.epi.out_recip = epi->out_recip; p.epi.mid_type = epi->mid_type;
    p.epi.bias_type = epi->bias_type; p.epi.col_scale = epi->col_scale; p.epi.bias = epi->bias;
    p.epi.clip_lo = epi->clip_lo; p.epi.clip_hi = epi->clip_hi; p.epi.in_zero = epi->in_zero;
    p.epi.out_zero = (epi->flags & RB_EPI_ZP_OUT) ? epi->out_zero : 0;
    p.epi.residual = epi->residual; p.epi.res_type = epi->res_type;
    p.epi.unary = (epi->flags & RB_EPI_UNARY) ? epi->unary : 0;
  } else if (p.out_type != (c.is_bf16 ? RB_BF16 : RB_F16)) {
    return fail(RB_UNSUPPORTED, "halo kernel: a converted result needs an epilogue");
  }
  p.status = dev->status_word;
  p.wait_cycles = kWaitCycles;
  p.wide_store = reinterpret_cast<uintptr_t>(out) % 32 == 0 && (c.o_n * 2) % 32 == 0 && (c.o_p * 2) % 32 == 0 && (c.o_q * 2) % 32 == 0;

  memset(&maps, 0, sizeof(maps));
  std::string err;
  const CUtensorMapDataType dt = c.is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  {
    const uint64_t dims[4] = {(uint64_t)c.C, (uint64_t)c.W, (uint64_t)c.H, (uint64_t)c.N};
    const uint64_t strides[3] = {(uint64_t)c.C * 2, (uint64_t)c.W * c.C * 2, (uint64_t)c.H * c.W * c.C * 2};
    const uint32_t box[4] = {64u, (uint32_t)p.Wp, (uint32_t)p.rows_box, 1u};
    if (!encode_tiled(&maps.in, dt, 4, image, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "halo kernel, image: " + err);
  }
  if (c.b_mn) {
    // the filter tensor [Kfil][FY][FX][Kout channels] with its own strides; one box = 64 k x 64 channels of one tap
    const uint64_t dims[4] = {(uint64_t)c.Kout, (uint64_t)c.FX, (uint64_t)c.FY, (uint64_t)c.C};
    const uint64_t strides[3] = {(uint64_t)c.f_sx * 2, (uint64_t)c.f_sy * 2, (uint64_t)c.f_sk * 2};
    const uint32_t box[4] = {64u, 1u, 1u, 64u};
    if (!encode_tiled(&maps.fil, dt, 4, filter_matrix, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "halo kernel, filter tensor: " + err);
  } else {
    const uint64_t ktot = (uint64_t)c.Y * c.X * c.C;
    const uint64_t dims[3] = {ktot, (uint64_t)c.Kout, 1};
    const uint64_t strides[2] = {ktot * 2, ktot * c.Kout * 2};
    const uint32_t box[3] = {64u, (uint32_t)c.Kout, 1u};
    if (!encode_tiled(&maps.fil, dt, 3, filter_matrix, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "halo kernel, filter: " + err);
  }
  *smem = p.stages * p.stage_bytes + fixed + 1024;
  return RB_SUCCESS;
}

// Rough cycles of one tile: its MMAs (shared-memory bound: 128 rows of A and Kout rows of B, 32 bytes each, per MMA at
// about 100 bytes per clock) or its epilogue, whichever is longer. Only the RATIO between the members of a group matters.
long long halo_tile_cost(const HaloParams& p) {
  const long long mma = (long long)p.G * p.Y * p.X * p.cchunks * 4 * ((4096 + p.Kout * 32) / 100) + 450;
  const long long epilogue = (long long)p.G * (p.Kout / 32) * 480 + 100;
  return std::max(mma, epilogue);
}

}  // namespace

RbStatus conv_halo_run(const HaloConv& c, const void* image, const void* filter_matrix, void* out, void* stream_v,
                       const RbEpilogue* epi, int out_type) {
  const void* filters[1] = {filter_matrix};
  void* outs[1] = {out};
  return conv_halo_run_group(&c, 1, image, filters, outs, stream_v, epi, out_type);
}

RbStatus conv_halo_run_group(const HaloConv* cs, int count, const void* image, const void* const* filter_matrices,
                             void* const* outs, void* stream_v, const RbEpilogue* epi, int out_type) {
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  if (count < 1 || count > kHaloMaxGroup) return fail(RB_UNSUPPORTED, "halo kernel: one to four convolutions per launch");
  HaloGroup g;
  memset(&g, 0, sizeof(g));
  g.n = count;
  int smem = 0;
  long long total_tiles = 0;
  for (int i = 0; i < count; ++i) {
    int sm = 0;
    RbStatus st = halo_setup(cs[i], image, filter_matrices[i], outs[i], epi, out_type, dev, g.prm[i], g.maps[i], &sm);
    if (st != RB_SUCCESS) return st;
    smem = std::max(smem, sm);
    total_tiles += g.prm[i].num_tiles;
  }
  // CTAs per member: one each, then one at a time to the member that would finish last
  int ctas[kHaloMaxGroup] = {0, 0, 0, 0};
  int grid = (int)std::min<long long>(total_tiles, dev->sm_count);
  if (grid < count) grid = count;
  for (int i = 0; i < count; ++i) ctas[i] = 1;
  for (int used = count; used < grid; ++used) {
    int worst = -1;
    long long worst_t = -1;
    for (int i = 0; i < count; ++i) {
      if (ctas[i] >= g.prm[i].num_tiles) continue;
      const long long t = (g.prm[i].num_tiles + ctas[i] - 1) / ctas[i] * halo_tile_cost(g.prm[i]);
      if (t > worst_t) { worst_t = t; worst = i; }
    }
    if (worst < 0) { grid = used; break; }
    ++ctas[worst];
  }
  for (int i = 0; i < count; ++i) g.first_cta[i + 1] = g.first_cta[i] + ctas[i];
  for (int i = count; i < kHaloMaxGroup; ++i) g.first_cta[i + 1] = g.first_cta[count];
  grid = g.first_cta[count];

  const bool with_epi = g.prm[0].epi.flags != 0;
  const void* kern = with_epi ? reinterpret_cast<const void*>(conv_halo_kernel<true>) : reinterpret_cast<const void*>(conv_halo_kernel<false>);
  RbStatus st = ensure_dynamic_smem(kern, smem);
  if (st != RB_SUCCESS) return st;
  unsigned long long* trace = trace_buffer((size_t)grid * 16);
  for (int i = 0; i < count; ++i) g.prm[i].trace = trace;
  if (with_epi) conv_halo_kernel<true><<<grid, kHaloThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(g);
  else conv_halo_kernel<false><<<grid, kHaloThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(g);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  return RB_SUCCESS;
}

}  // namespace rb
