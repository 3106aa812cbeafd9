// Backward weight of a unit-stride NHWC convolution without an im2col matrix and without re-reading the input once
// per filter tap.
//
// rocMLIR lowers rock.conv_bwd_weight to a GEMM whose reduction runs over the output pixels
// (ConvRewritePattern / backwardWeightAtomicAdd, mlir/lib/Dialect/Rock/Transforms/ConvToGemm.cpp:520-760): the filter
// gradient dW[k][(y, x, c)] = sum over pixels of dY[pixel][k] * X[pixel shifted by the tap][c], split along the pixels
// with an atomic add of the partial sums. The im2col-TMA form of this library fetches the shifted input tile of every
// tap from L2 again. This kernel fetches, per tile of R output rows of one image,
//
//   * the input window WITH ITS HALO once (one tiled TMA load per 64-channel block: [rows][Wp] pixels of 128 bytes,
//     zero outside the image), and
//   * the output-gradient rows on the same padded raster m = r * Wp + q (columns q >= Q and rows past the image are
//     outside the tensor, so the load fills them with zeros and they add nothing);
//
// both operands are "MN-major" for the tensor core: a shared-memory row is one pixel (one step of the reduction) and
// holds 64 contiguous channels. The A operand of tap (y, x) is the window shifted by y * dil_h * Wp + x * dil_w rows:
// only the descriptor's start address changes (the 128-byte swizzle follows absolute address bits). Two taps share one
// M = 128 MMA: the descriptor's leading-dimension offset, the distance between the two 64-channel halves of A, is simply
// the distance between the two taps' windows. The accumulators of all taps stay in tensor memory for the whole kernel;
// at the end every CTA stores its partial sums as one f32 slab (coalesced: lanes of a warp are neighbours in a row of
// dW) and a second, small kernel adds the slabs and converts to the 16-bit filter gradient (atomic adds of 148 CTAs
// into one buffer were measured several times slower than the MMAs of a small problem). Filters whose accumulators
// exceed the 512 TMEM columns are divided among groups of CTAs (each group walks all pixels for its share of the taps).
//
// Non-finite inputs: a zero of the padded raster multiplies whatever pixel the shifted window holds there, so an Inf
// or NaN in the input can reach taps that the reference's gather would not pair it with.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <string>

#include "lib_state.h"
#include "ptx.cuh"

namespace rb {
namespace {

constexpr int kWgThreads = 256;
constexpr int kWgMaxStages = 6;
constexpr int kWgMaxPairs = 32;
constexpr int kWgSlack = 160 * 128;   // rows that shifted descriptors may touch past the last stage

struct WgradMaps {
  CUtensorMap x;    // {C, W, H, N} of the NHWC input, box {64, Wp, rows_box, 1}
  CUtensorMap dy;   // {Kout, Q, P, N} of the NHWK output gradient, box {64, Wp, R, 1}
};

struct WgradParams {
  int Kout, cchunks, kchunks, yxc;
  int pad_h, pad_w;
  int Wp, R, ksteps;                 // padded raster width, output rows per tile, 16-pixel reduction steps per tile
  int tiles_per_img, num_tiles;
  int x_plane_bytes, dy_plane_bytes, x_box_bytes, dy_box_bytes, stage_bytes, stages;
  int npairs, pairs_per_cta, groups;
  uint32_t idesc;
  int is_bf16;
  float* slabs;                      // [ctas of a group][Kout][Y * X * C] partial sums (each CTA writes its share of the columns)
  uint32_t* status;
  long long wait_cycles;
  unsigned long long* trace;         // optional [gridDim.x][16]: [2] MMA warp waited for a stage, [4] its loop, [5] tiles
  uint32_t pair_off[kWgMaxPairs];    // (byte offset of the pair's first window from the stage base) >> 4
  uint32_t pair_lbo[kWgMaxPairs];    // (distance between the pair's two windows) >> 4
  int pair_col0[kWgMaxPairs];        // column (tap * C + channel block * 64) of either half in a row of dW; -1 = unused
  int pair_col1[kWgMaxPairs];
};

__global__ void __launch_bounds__(kWgThreads, 1)
conv_wgrad_halo_kernel(const __grid_constant__ WgradMaps maps, const __grid_constant__ WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int ring_bytes = p.stages * p.stage_bytes + kWgSlack;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ring_bytes);
  uint64_t* full_bar = bars;                     // [stages]
  uint64_t* empty_bar = bars + kWgMaxStages;     // [stages]
  uint64_t* done_bar = bars + 2 * kWgMaxStages;  // [1]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kWgMaxStages + 1);
  const int warp = warp_id_uniform();
  const long long wait_limit = p.wait_cycles;

  // this CTA's share: group = a slice of the tap pairs, rank within the group = a slice of the tiles
  const int group = (int)blockIdx.x % p.groups;
  const int cta = (int)blockIdx.x / p.groups;
  const int ctas = ((int)gridDim.x - group + p.groups - 1) / p.groups;
  const int pair0 = group * p.pairs_per_cta;
  const int my_pairs = min(p.pairs_per_cta, p.npairs - pair0);
  const int my_tiles = cta < p.num_tiles ? (p.num_tiles - cta + ctas - 1) / ctas : 0;

  // The ring starts out as zeros: rows that no load ever writes (the tail of the gradient raster, the slack past the
  // last stage) are multiplied into the sums and must be finite / zero.
  {
    uint4* z = reinterpret_cast<uint4*>(smem);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < ring_bytes / 16; i += kWgThreads) z[i] = zero;
    fence_proxy_async();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(done_bar, 1);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<1>(tmem_holder, 512);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane_id() == 0) { prefetch_tmap(&maps.x); prefetch_tmap(&maps.dy); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane_id() == 0) {
      uint32_t s = 0, ph = 0;
      const uint32_t tx_bytes = (uint32_t)(p.cchunks * p.x_box_bytes + p.kchunks * p.dy_box_bytes);
      for (int tile = cta; tile < p.num_tiles; tile += ctas) {
        const int n = tile / p.tiles_per_img;
        const int p0 = (tile - n * p.tiles_per_img) * p.R;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, p.status, kStatusTimeoutProducer + s, wait_limit)) break;
        mbar_expect_tx(&full_bar[s], tx_bytes);
        uint8_t* st = smem + (size_t)s * p.stage_bytes;
        for (int cc = 0; cc < p.cchunks; ++cc)
          tma_load_4d(st + (size_t)cc * p.x_plane_bytes, &maps.x, &full_bar[s], cc * 64, -p.pad_w, p0 - p.pad_h, n);
        uint8_t* dy = st + (size_t)p.cchunks * p.x_plane_bytes;
        for (int kc = 0; kc < p.kchunks; ++kc)
          tma_load_4d(dy + (size_t)kc * p.dy_plane_bytes, &maps.dy, &full_bar[s], kc * 64, 0, p0, n);
        if (++s == (uint32_t)p.stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the loop (its counters and descriptor words are warp-uniform); one elected lane issues.
    // one lane, chosen once: the commits must come from the thread that issued the MMAs they track
    const bool leader = elect_one();
    const int ksteps = p.ksteps, Kout = p.Kout;
    const uint32_t stages = (uint32_t)p.stages, idesc = p.idesc;
    const bool tracing = p.trace != nullptr;
    const uint32_t desc_hi = smem_desc_hi(1024);
    const uint32_t x_lo0 = smem_desc_lo(smem_u32(smem), 0);
    const uint32_t dy_lo0 = smem_desc_lo(smem_u32(smem) + (uint32_t)(p.cchunks * p.x_plane_bytes), (uint32_t)p.dy_plane_bytes);
    const uint32_t stage_step = (uint32_t)p.stage_bytes >> 4;
    constexpr uint32_t kStep = (16 * 128) >> 4;   // sixteen pixels = sixteen 128-byte rows on
    uint32_t s = 0, ph = 0;
    long long w_full = 0;
    const long long t_begin = tracing ? clock64() : 0;
    bool ok = true;
    bool ready = false;
    for (int t = 0; t < my_tiles && ok; ++t) {
      if (!ready) {
        const long long tw = tracing ? clock64() : 0;
        if (!mbar_wait_warp(&full_bar[s], ph, p.status, kStatusTimeoutMma + s, wait_limit)) { ok = false; break; }
        if (tracing) w_full += clock64() - tw;
      }
      tc_fence_after();
      // the NEXT stage's barrier is tested before this tile's last reduction step is issued: the answer arrives while
      // those MMAs queue up, and the wait above is skipped when the stage is already full
      uint32_t ns = s + 1, nph = ph;
      if (ns == stages) { ns = 0; nph ^= 1u; }
      bool next_ready = false;
      const uint32_t x_lo = x_lo0 + s * stage_step;
      uint32_t dy_lo = dy_lo0 + s * stage_step;
      uint32_t koff = 0;
      for (int ks = 0; ks < ksteps; ++ks) {
        if (ks + 1 == ksteps) next_ready = __shfl_sync(0xffffffffu, mbar_test_wait(&full_bar[ns], nph) ? 1 : 0, 0) != 0;
        const uint64_t b_desc = desc64(dy_lo, desc_hi);
        const uint32_t accum = (t | ks) ? 1u : 0u;
        for (int j = 0; j < my_pairs; ++j) {
          const uint32_t a_lo = (x_lo + p.pair_off[pair0 + j] + koff) | (p.pair_lbo[pair0 + j] << 16);
          if (leader) umma_ss<kKindF16, 1>(tmem_base + (uint32_t)(j * Kout), desc64(a_lo, desc_hi), b_desc, idesc, accum);
        }
        dy_lo += kStep;
        koff += kStep;
      }
      if (leader) tc_commit_addr1(smem_u32(&empty_bar[s]));
      s = ns; ph = nph; ready = next_ready;
    }
    if (leader) tc_commit<1>(done_bar);
    if (tracing && lane_id() == 0) {
      p.trace[blockIdx.x * 16 + 2] = (unsigned long long)w_full;
      p.trace[blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - t_begin);
      p.trace[blockIdx.x * 16 + 5] = (unsigned long long)my_tiles;
    }
  } else if (warp >= 4) {
    // ------------------------------ final sums ------------------------------
    // TMEM lane = channel within the pair's two 64-channel halves, column = output channel k: lanes of a warp are
    // neighbours in a row of dW, so each store instruction covers 128 contiguous bytes of the CTA's slab. A CTA
    // without tiles stores zeros.
    const int q4 = warp & 3, lane = lane_id();
    const int row = q4 * 32 + lane;
    const bool have = my_tiles > 0 && mbar_wait_warp(done_bar, 0, p.status, kStatusTimeoutEpilogue, wait_limit);
    tc_fence_after();
    float* slab = p.slabs + (size_t)cta * p.Kout * p.yxc;
    for (int j = 0; j < my_pairs; ++j) {
      const int col = row < 64 ? p.pair_col0[pair0 + j] : p.pair_col1[pair0 + j];
      float* dst = slab + (col < 0 ? 0 : col) + (row & 63);
#pragma unroll 1
      for (int k0 = 0; k0 < p.Kout; k0 += 32) {
        uint32_t v[32];
        if (have) {
          tmem_ld32(tmem_base + (uint32_t(q4 * 32) << 16) + (uint32_t)(j * p.Kout + k0), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (col >= 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[(size_t)(k0 + i) * p.yxc] = __uint_as_float(v[i]);
        }
      }
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

// Adds the slabs and converts: a block covers 32 float4 columns x 8 slices of the slabs (eight independent 16-byte
// loads in flight per thread); the slices meet in shared memory.
__global__ void __launch_bounds__(256)
conv_wgrad_sum_kernel(const float* __restrict__ slabs, int nslabs, int elems, void* __restrict__ out, int is_bf16) {
  __shared__ float4 part[8][32];
  const int lane4 = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int i4 = blockIdx.x * 32 + lane4;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i4 * 4 < elems) {
    const float4* src = reinterpret_cast<const float4*>(slabs) + i4;
    const size_t stride4 = (size_t)elems / 4;
    int s = slice;
    for (; s + 56 < nslabs; s += 64) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(src + (size_t)(s + 8 * u) * stride4);
#pragma unroll
      for (int u = 0; u < 8; ++u) { a.x += v[u].x; a.y += v[u].y; a.z += v[u].z; a.w += v[u].w; }
    }
    for (; s < nslabs; s += 8) {
      const float4 v = __ldcg(src + (size_t)s * stride4);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
  }
  part[slice][lane4] = a;
  __syncthreads();
  if (slice == 0 && i4 * 4 < elems) {
#pragma unroll
    for (int s = 1; s < 8; ++s) { const float4 v = part[s][lane4]; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
    uint2 w;
    if (is_bf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
      w.x = *reinterpret_cast<uint32_t*>(&lo); w.y = *reinterpret_cast<uint32_t*>(&hi);
    } else {
      __half2 lo = __floats2half2_rn(a.x, a.y), hi = __floats2half2_rn(a.z, a.w);
      w.x = *reinterpret_cast<uint32_t*>(&lo); w.y = *reinterpret_cast<uint32_t*>(&hi);
    }
    reinterpret_cast<uint2*>(out)[i4] = w;
  }
}

struct WgradShape {
  int Wp, R, rows_box, ksteps, cchunks, kchunks, units, npairs, pairs_per_cta, groups;
  int x_plane_bytes, dy_plane_bytes, stage_bytes, stages;
};

// Units in (tap, channel block) order; consecutive units share an MMA: the half at the lower address comes first and
// the leading-dimension offset is the (positive) distance to the other. False when a distance does not fit the
// descriptor's 14-bit field.
bool wgrad_pairs(const HaloConv& c, const WgradShape& s, uint32_t* off, uint32_t* lbo, int* col0, int* col1) {
  for (int u = 0; u < s.units; u += 2) {
    long long o[2] = {0, 0};
    int col[2] = {-1, -1};
    for (int h = 0; h < 2 && u + h < s.units; ++h) {
      const int tap = (u + h) / s.cchunks, cc = (u + h) % s.cchunks;
      const int y = tap / c.X, x = tap % c.X;
      o[h] = (long long)cc * s.x_plane_bytes + ((long long)y * c.dil_h * s.Wp + (long long)x * c.dil_w) * 128;
      col[h] = tap * c.C + cc * 64;
    }
    const bool lone = u + 1 >= s.units;
    const int first = (lone || o[0] < o[1]) ? 0 : 1;
    const long long d = lone ? 0 : o[1 - first] - o[first];
    if (!lone && (d <= 0 || (d >> 4) >= 0x4000)) return false;
    if (off) {
      off[u / 2] = (uint32_t)(o[first] >> 4);
      lbo[u / 2] = (uint32_t)(d >> 4);
      col0[u / 2] = col[first];
      col1[u / 2] = lone ? -1 : col[1 - first];
    }
  }
  return true;
}

bool wgrad_shape(const HaloConv& c, WgradShape* s) {
  if (c.C % 64 || c.Kout % 64 || c.Kout > 256 || c.Kout < 64) return false;
  if (c.dil_h < 1 || c.dil_w < 1 || c.pad_h < 0 || c.pad_w < 0 || c.Y * c.X > 49) return false;
  s->Wp = c.Q + (c.X - 1) * c.dil_w;
  if (s->Wp > 128 || s->Wp != c.W + c.pad_w + c.pad_w_r) return false;
  if (c.P + (c.Y - 1) * c.dil_h != c.H + c.pad_h + c.pad_h_r) return false;
  s->cchunks = c.C / 64;
  s->kchunks = c.Kout / 64;
  // Output rows per tile: the reduction runs along the raster, so a tile may be any number of rows long. More rows
  // share the window's halo rows and waste less of the last 16-pixel step; the ring must still hold three stages.
  // Among the sizes that fit, the one with the fewest reduction steps per image wins.
  int best_r = 0;
  long long best_steps = 0;
  for (int r = 1; r <= std::min(c.P, 16); ++r) {
    const int rows_box = r + (c.Y - 1) * c.dil_h;
    const int ksteps = (r * s->Wp + 15) / 16;
    const long long stage = (long long)s->cchunks * ((s->Wp * rows_box + 7) / 8 * 8 * 128) + (long long)s->kchunks * ksteps * 16 * 128;
    if (rows_box > 256 || (232448 - 1024 - kWgSlack - 1024) / stage < 3) continue;
    const long long steps = (long long)((c.P + r - 1) / r) * (ksteps + 2);   // + the barrier work of a tile, about two steps' worth
    if (best_r == 0 || steps <= best_steps) { best_r = r; best_steps = steps; }
  }
  if (best_r == 0) {   // not even one row with three stages: two stages of the 128-row tile, as before
    best_r = std::min(128 / s->Wp, c.P);
  }
  s->R = best_r;
  s->rows_box = s->R + (c.Y - 1) * c.dil_h;
  if (s->R < 1 || s->rows_box > 256) return false;
  s->ksteps = (s->R * s->Wp + 15) / 16;
  s->units = c.Y * c.X * s->cchunks;
  s->npairs = (s->units + 1) / 2;
  if (s->npairs > kWgMaxPairs) return false;
  s->pairs_per_cta = std::min(s->npairs, 512 / c.Kout);
  s->groups = (s->npairs + s->pairs_per_cta - 1) / s->pairs_per_cta;
  s->x_plane_bytes = (s->Wp * s->rows_box + 7) / 8 * 8 * 128;
  s->dy_plane_bytes = s->ksteps * 16 * 128;
  s->stage_bytes = s->cchunks * s->x_plane_bytes + s->kchunks * s->dy_plane_bytes;
  s->stages = std::min(kWgMaxStages, (232448 - 1024 - kWgSlack - 1024) / s->stage_bytes);
  return s->stages >= 2 && wgrad_pairs(c, *s, nullptr, nullptr, nullptr, nullptr);
}

}  // namespace

bool conv_wgrad_halo_applicable(const HaloConv& c) {
  WgradShape s;
  return wgrad_shape(c, &s);
}

namespace {
// CTAs of the launch: whole groups (every slice of the taps sees every tile), at least four tiles per CTA when the
// problem is small (every CTA adds a slab to the final sum).
int wgrad_grid(const HaloConv& c, const WgradShape& s, int sm_count) {
  const long long tiles = (long long)c.N * ((c.P + s.R - 1) / s.R);
  const long long per_group = std::max<long long>(1, std::min<long long>(sm_count / s.groups, (tiles + 3) / 4));
  return (int)per_group * s.groups;
}
}  // namespace

size_t conv_wgrad_halo_workspace(const HaloConv& c) {
  WgradShape s;
  const DeviceInfo* dev = device_info();
  if (!dev || !wgrad_shape(c, &s)) return 0;
  return (size_t)(wgrad_grid(c, s, dev->sm_count) / s.groups) * c.Kout * c.Y * c.X * c.C * sizeof(float);
}

RbStatus conv_wgrad_halo_run(const HaloConv& c, const void* image, const void* out_grad, void* filter_grad, void* workspace,
                             size_t workspace_bytes, void* stream_v) {
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  WgradShape s;
  if (!wgrad_shape(c, &s)) return fail(RB_UNSUPPORTED, "convolution outside the reach of the halo weight-gradient kernel");
  const size_t need = conv_wgrad_halo_workspace(c);
  if (!workspace || workspace_bytes < need) return fail(RB_WORKSPACE_TOO_SMALL, "halo weight-gradient kernel: workspace too small");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  WgradParams p;
  memset(&p, 0, sizeof(p));
  p.Kout = c.Kout; p.cchunks = s.cchunks; p.kchunks = s.kchunks; p.yxc = c.Y * c.X * c.C;
  p.pad_h = c.pad_h; p.pad_w = c.pad_w;
  p.Wp = s.Wp; p.R = s.R; p.ksteps = s.ksteps;
  p.tiles_per_img = (c.P + s.R - 1) / s.R;
  p.num_tiles = c.N * p.tiles_per_img;
  p.x_plane_bytes = s.x_plane_bytes; p.dy_plane_bytes = s.dy_plane_bytes;
  p.x_box_bytes = s.Wp * s.rows_box * 128; p.dy_box_bytes = s.Wp * s.R * 128;
  p.stage_bytes = s.stage_bytes; p.stages = s.stages;
  p.npairs = s.npairs; p.pairs_per_cta = s.pairs_per_cta; p.groups = s.groups;
  const uint32_t fmt = c.is_bf16 ? 1u : 0u;
  p.idesc = make_idesc(1, fmt, fmt, 1, 1, 128, (uint32_t)c.Kout);
  p.is_bf16 = c.is_bf16;
  p.slabs = static_cast<float*>(workspace);
  p.status = dev->status_word;
  p.wait_cycles = kWaitCycles;
  if (!wgrad_pairs(c, s, p.pair_off, p.pair_lbo, p.pair_col0, p.pair_col1))
    return fail(RB_UNSUPPORTED, "halo weight-gradient kernel: taps too far apart");

  WgradMaps maps;
  memset(&maps, 0, sizeof(maps));
  std::string err;
  const CUtensorMapDataType dt = c.is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  {
    const uint64_t dims[4] = {(uint64_t)c.C, (uint64_t)c.W, (uint64_t)c.H, (uint64_t)c.N};
    const uint64_t strides[3] = {(uint64_t)c.C * 2, (uint64_t)c.W * c.C * 2, (uint64_t)c.H * c.W * c.C * 2};
    const uint32_t box[4] = {64u, (uint32_t)s.Wp, (uint32_t)s.rows_box, 1u};
    if (!encode_tiled(&maps.x, dt, 4, image, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "halo weight-gradient kernel, input: " + err);
  }
  {
    const uint64_t dims[4] = {(uint64_t)c.Kout, (uint64_t)c.Q, (uint64_t)c.P, (uint64_t)c.N};
    const uint64_t strides[3] = {(uint64_t)c.Kout * 2, (uint64_t)c.Q * c.Kout * 2, (uint64_t)c.P * c.Q * c.Kout * 2};
    const uint32_t box[4] = {64u, (uint32_t)s.Wp, (uint32_t)s.R, 1u};
    if (!encode_tiled(&maps.dy, dt, 4, out_grad, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "halo weight-gradient kernel, output gradient: " + err);
  }
  const int smem = s.stages * s.stage_bytes + kWgSlack + 1024 + 1024;
  RbStatus st = ensure_dynamic_smem(reinterpret_cast<const void*>(conv_wgrad_halo_kernel), smem);
  if (st != RB_SUCCESS) return st;
  const int grid = wgrad_grid(c, s, dev->sm_count);
  p.trace = trace_buffer((size_t)grid * 16);
  conv_wgrad_halo_kernel<<<grid, kWgThreads, smem, stream>>>(maps, p);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  const int elems = c.Kout * p.yxc;
  conv_wgrad_sum_kernel<<<(elems / 4 + 31) / 32, 256, 0, stream>>>(p.slabs, grid / s.groups, elems, filter_grad, c.is_bf16);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  return RB_SUCCESS;
}

}  // namespace rb
