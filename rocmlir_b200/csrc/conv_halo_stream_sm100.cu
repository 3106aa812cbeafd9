// Halo convolution with a STREAMED filter: the forward form of csrc/conv_halo_sm100.cu for filters that do not fit
// into shared memory beside the window ring, and for f32 tensors.
//
// Same idea as the resident-filter kernel (rocMLIR's implicit GEMM, ConvToGemm.cpp:1133-1400, re-reads the shifted
// input window once per filter tap; here an output tile's window is loaded once with its halo and every tap is a
// shifted view of it), but the filter matrix B[k][(y, x, c)] travels through its own ring of shared-memory slabs, one
// (tap, channel block) slab of Kout rows x 128 bytes at a time, in the order the MMAs consume them. A slab is used by
// every sub-tile of the stage before it is released, so the window pays for itself G times.
//
// f32 tensors run as three TF32 products per step - hi.hi, and lo.hi + hi.lo into a second accumulator that the
// epilogue adds, with x = hi + lo split exactly into TF32 parts (the split the GEMM kernel uses, csrc/gemm_sm100.cu f32_planes) - from TWO window planes and TWO filter
// planes that are loaded once per stage / slab; the im2col form loads both operands again for each of the three
// products of every K block (72 KB where 48 KB of distinct data exist) and once per tap on top of that.
//
// Roles: warp 0 producer (windows and slabs, one FIFO order), warp 1 MMA issuer (all lanes run the loop, one lane
// elected once issues), warp 2 TMEM allocator, warps 4-7 / 8-11 two epilogue groups (one per accumulator buffer).
// Every wait is bounded and reports through the device status word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <string>

#include "lib_state.h"
#include "ptx.cuh"

namespace rb {
namespace {

constexpr int kStThreads = 384;
constexpr int kStMaxW = 4;    // window stages
constexpr int kStMaxB = 8;    // filter-slab stages

struct StreamMaps {
  CUtensorMap in[2];    // {C, W, H, N} of the NHWC image (f32: hi and lo TF32 planes), box {128 bytes of channels, Wp, rows_box, 1}
  CUtensorMap fil[2];   // {Y * X * C, Kout, 1} of the K-major filter matrix (f32: hi and lo planes), box {128 bytes, Kout, 1}
};

struct StreamParams {
  int N, P, Q, Kout, cchunks, epr;      // epr = elements per 128-byte row: 64 (16-bit) or 32 (f32)
  int Y, X, dil_h, dil_w, pad_h, pad_w;
  int Wp, R, rows_box, G;
  int tiles_per_img, num_tiles;
  int planes;                            // 1, or 2 for f32 (hi, lo)
  int win_bytes, wstages;                // one plane of one window stage; a stage holds `planes` of them
  int slab_bytes, bstages;               // one plane of one filter slab
  int slack_bytes;
  uint32_t idesc;
  int is_bf16;
  void* out;
  long long o_n, o_p, o_q, o_k;          // element strides of (image, row, column, channel) in the result
  uint32_t* status;
  long long wait_cycles;
  unsigned long long* trace;             // optional [gridDim.x][16]: [2] waited for windows, [3] for slabs, [4] MMA loop, [5] tiles
};

template <bool F32>
__global__ void __launch_bounds__(kStThreads, 1)
conv_halo_stream_kernel(const __grid_constant__ StreamMaps maps, const __grid_constant__ StreamParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int PL = F32 ? 2 : 1;
  const int wstage_bytes = PL * p.win_bytes, bstage_bytes = PL * p.slab_bytes;
  uint8_t* b_smem = smem + p.wstages * wstage_bytes + p.slack_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_smem + p.bstages * bstage_bytes);
  uint64_t* wfull = bars;                       // [kStMaxW]
  uint64_t* wempty = bars + kStMaxW;            // [kStMaxW]
  uint64_t* bfull = bars + 2 * kStMaxW;         // [kStMaxB]
  uint64_t* bempty = bars + 2 * kStMaxW + kStMaxB;
  uint64_t* tfull = bars + 2 * kStMaxW + 2 * kStMaxB;   // [2]
  uint64_t* tempty = tfull + 2;                          // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  const int warp = warp_id_uniform();
  const long long wait_limit = p.wait_cycles;
  const int cta = (int)blockIdx.x, ctas = (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.wstages; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], 1); }
    for (int s = 0; s < p.bstages; ++s) { mbar_init(&bfull[s], 1); mbar_init(&bempty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4); }
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc<1>(tmem_holder, 512);
    tmem_relinquish<1>();
  }
  if (warp == 0 && lane_id() == 0) {
    for (int i = 0; i < PL; ++i) { prefetch_tmap(&maps.in[i]); prefetch_tmap(&maps.fil[i]); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int taps = p.Y * p.X;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane_id() == 0) {
      uint32_t ws = 0, wph = 0, bs = 0, bph = 0;
      bool ok = true;
      const uint32_t win_tx = (uint32_t)(PL * p.Wp * p.rows_box * 128), slab_tx = (uint32_t)(PL * p.slab_bytes);
      for (int tile = cta; ok && tile < p.num_tiles; tile += ctas) {
        const int n = tile / p.tiles_per_img;
        const int p0 = (tile - n * p.tiles_per_img) * p.R * p.G;
        for (int cc = 0; cc < p.cchunks && ok; ++cc) {
          if (!mbar_wait(&wempty[ws], wph ^ 1u, p.status, kStatusTimeoutProducer + ws, wait_limit)) { ok = false; break; }
          mbar_expect_tx(&wfull[ws], win_tx);
          for (int pl = 0; pl < PL; ++pl)
            tma_load_4d(smem + (size_t)ws * wstage_bytes + (size_t)pl * p.win_bytes, &maps.in[pl], &wfull[ws], cc * p.epr, -p.pad_w,
                        p0 - p.pad_h, n);
          if (++ws == (uint32_t)p.wstages) { ws = 0; wph ^= 1u; }
          for (int tap = 0; tap < taps; ++tap) {
            if (!mbar_wait(&bempty[bs], bph ^ 1u, p.status, kStatusTimeoutProducer + 0x10 + bs, wait_limit)) { ok = false; break; }
            mbar_expect_tx(&bfull[bs], slab_tx);
            for (int pl = 0; pl < PL; ++pl)
              tma_load_3d(b_smem + (size_t)bs * bstage_bytes + (size_t)pl * p.slab_bytes, &maps.fil[pl], &bfull[bs],
                          (tap * p.cchunks + cc) * p.epr, 0, 0);
            if (++bs == (uint32_t)p.bstages) { bs = 0; bph ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    const bool leader = elect_one();   // one lane, chosen once: commits must come from the thread whose MMAs they track
    const int Y = p.Y, X = p.X, cchunks = p.cchunks, num_tiles = p.num_tiles, G = p.G, Kout = p.Kout;
    const uint32_t wstages = (uint32_t)p.wstages, bstages = (uint32_t)p.bstages, idesc = p.idesc;
    const bool tracing = p.trace != nullptr;
    uint32_t* const status = p.status;
    const uint32_t desc_hi = smem_desc_hi(1024);
    const uint32_t a_xstep = (uint32_t)p.dil_w * 8u, a_ystep = (uint32_t)(p.dil_h * p.Wp) * 8u;
    const uint32_t g_step = (uint32_t)(p.R * p.Wp) * 8u;
    const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), 16), b_lo0 = smem_desc_lo(smem_u32(b_smem), 16);
    const uint32_t w_step = (uint32_t)wstage_bytes >> 4, b_step = (uint32_t)bstage_bytes >> 4;
    const uint32_t a_plane = (uint32_t)p.win_bytes >> 4, b_plane = (uint32_t)p.slab_bytes >> 4;
    uint32_t ws = 0, wph = 0, bs = 0, bph = 0, t = 0;
    long long w_win = 0, w_slab = 0;
    const long long t_begin = tracing ? clock64() : 0;
    bool ok = true;
    for (int tile = cta; ok && tile < num_tiles; tile += ctas, ++t) {
      const uint32_t buf = t & 1u, tph = (t >> 1) & 1u;
      if (!mbar_wait_warp(&tempty[buf], tph ^ 1u, status, kStatusTimeoutMma + 0x10 + buf, wait_limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * 256;
      for (int cc = 0; cc < cchunks && ok; ++cc) {
        const long long tw = tracing ? clock64() : 0;
        if (!mbar_wait_warp(&wfull[ws], wph, status, kStatusTimeoutMma + ws, wait_limit)) { ok = false; break; }
        if (tracing) w_win += clock64() - tw;
        const uint32_t a_base = a_lo0 + ws * w_step;
        uint32_t a_row = a_base;
        for (int y = 0; y < Y && ok; ++y) {
          uint32_t a_tap = a_row;
          for (int x = 0; x < X; ++x) {
            const long long tb = tracing ? clock64() : 0;
            if (!mbar_wait_warp(&bfull[bs], bph, status, kStatusTimeoutMma + 0x20 + bs, wait_limit)) { ok = false; break; }
            if (tracing) w_slab += clock64() - tb;
            tc_fence_after();
            const uint32_t b_lo = b_lo0 + bs * b_step;
            if (leader) {
              const uint32_t first = (cc | y | x) ? 1u : 0u;   // the tile's first tap overwrites the accumulator
              for (int gsub = 0; gsub < G; ++gsub) {
                const uint32_t a_lo = a_tap + (uint32_t)gsub * g_step;
                const uint32_t d = tmem_d + (uint32_t)(gsub * Kout);
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // 128 bytes of channels = four K steps
                  if constexpr (F32) {
                    // the two small products go to an accumulator of their own (added to the main one in the epilogue):
                    // summed into the hi.hi accumulator they would be truncated against a value 2^11 times their size
                    const uint32_t ds = d + (uint32_t)(G * Kout);
                    umma_ss<kKindTF32, 1>(ds, desc64(a_lo + a_plane + k * 2, desc_hi), desc64(b_lo + k * 2, desc_hi), idesc, k ? 1u : first);   // lo . hi
                    umma_ss<kKindTF32, 1>(ds, desc64(a_lo + k * 2, desc_hi), desc64(b_lo + b_plane + k * 2, desc_hi), idesc, 1u);               // hi . lo
                    umma_ss<kKindTF32, 1>(d, desc64(a_lo + k * 2, desc_hi), desc64(b_lo + k * 2, desc_hi), idesc, k ? 1u : first);              // hi . hi
                  } else {
                    umma_ss<kKindF16, 1>(d, desc64(a_lo + k * 2, desc_hi), desc64(b_lo + k * 2, desc_hi), idesc, k ? 1u : first);
                  }
                }
              }
              tc_commit_addr1(smem_u32(&bempty[bs]));
            }
            if (++bs == bstages) { bs = 0; bph ^= 1u; }
            a_tap += a_xstep;
          }
          a_row += a_ystep;
        }
        if (leader) tc_commit_addr1(smem_u32(&wempty[ws]));
        if (++ws == wstages) { ws = 0; wph ^= 1u; }
      }
      if (!ok) break;
      if (leader) tc_commit<1>(&tfull[buf]);
    }
    if (tracing && lane_id() == 0) {
      p.trace[blockIdx.x * 16 + 2] = (unsigned long long)w_win;
      p.trace[blockIdx.x * 16 + 3] = (unsigned long long)w_slab;
      p.trace[blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - t_begin);
      p.trace[blockIdx.x * 16 + 5] = t;
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue: two groups, one per accumulator buffer ------------------------------
    const int q4 = warp & 3, lane = lane_id();
    const uint32_t egroup = (uint32_t)(warp - 4) >> 2;
    const int m = q4 * 32 + lane;              // position on the sub-tile's padded raster
    const int Wp = p.Wp, R = p.R, P = p.P, Q = p.Q, Kout = p.Kout, tiles_per_img = p.tiles_per_img, num_tiles = p.num_tiles, G = p.G;
    const long long o_n = p.o_n, o_p = p.o_p, o_q = p.o_q, o_k = p.o_k;
    const bool is_bf16 = p.is_bf16 != 0;
    const int rr = m / Wp, qq = m - rr * Wp;
    uint32_t t = 0;
    for (int tile = cta; tile < num_tiles; tile += ctas, ++t) {
      const uint32_t buf = t & 1u, tph = (t >> 1) & 1u;
      if (buf != egroup) continue;
      if (!mbar_wait_warp(&tfull[buf], tph, p.status, kStatusTimeoutEpilogue + buf, wait_limit)) break;
      tc_fence_after();
      const int n = tile / tiles_per_img;
      for (int gsub = 0; gsub < G; ++gsub) {
        const int p0 = (tile - n * tiles_per_img) * R * G + gsub * R;
        const bool valid = rr < R && qq < Q && p0 + rr < P;
        const long long pix = (long long)n * o_n + (long long)(p0 + rr) * o_p + (long long)qq * o_q;   // elements
        const uint32_t taddr = tmem_base + (uint32_t(q4 * 32) << 16) + buf * 256 + (uint32_t)(gsub * Kout);
#pragma unroll 1
        for (int c = 0; c < Kout; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          if constexpr (F32) {
            uint32_t u[32];
            tmem_ld32(taddr + (uint32_t)(G * Kout) + c, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), __uint_as_float(u[j])));
          } else {
            tmem_ld_wait();
          }
          if (!valid) continue;
          if constexpr (F32) {
            float* dst = static_cast<float*>(p.out) + pix + (long long)c * o_k;
            if (o_k == 1) {   // channels last: 128 contiguous bytes per thread
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {          // channel planes (NKHW): neighbouring lanes are neighbouring pixels of a plane
#pragma unroll
              for (int j = 0; j < 32; ++j) dst[(long long)j * o_k] = __uint_as_float(v[j]);
            }
          } else {
            uint32_t h[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float lo = __uint_as_float(v[2 * j]), hi = __uint_as_float(v[2 * j + 1]);
              if (is_bf16) { __nv_bfloat162 t2 = __floats2bfloat162_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
              else { __half2 t2 = __floats2half2_rn(lo, hi); h[j] = *reinterpret_cast<uint32_t*>(&t2); }
            }
            uint8_t* dst = static_cast<uint8_t*>(p.out) + 2 * (pix + c);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + i * 16) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
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

struct StreamShape {
  int Wp, R, G, rows_box, win_bytes, slab_bytes, wstages, bstages, slack_bytes, cchunks, epr;
};

bool stream_shape(const HaloConv& c, int elem_bytes, long long o_k, StreamShape* s) {
  const int planes = elem_bytes == 4 ? 2 : 1;
  s->epr = 128 / elem_bytes;
  if (c.b_mn || c.C % s->epr || c.Kout % 32 || c.Kout > 256 || c.Kout < 32) return false;
  if (elem_bytes == 2 && o_k != 1) return false;   // 16-bit results are stored channels-last only
  if (c.dil_h < 1 || c.dil_w < 1 || c.pad_h < 0 || c.pad_w < 0 || c.Y * c.X > 49) return false;
  s->Wp = c.Q + (c.X - 1) * c.dil_w;
  if (s->Wp > 128 || s->Wp != c.W + c.pad_w + c.pad_w_r) return false;
  if (c.P + (c.Y - 1) * c.dil_h != c.H + c.pad_h + c.pad_h_r) return false;
  s->R = std::min(128 / s->Wp, c.P);
  if (s->R < 1) return false;
  s->cchunks = c.C / s->epr;
  s->slab_bytes = c.Kout * 128;
  // The rows of a 128-row MMA beyond R * Wp (shifted by the tap) lie past the end of the window: their results are
  // discarded and MMA rows do not mix, so they may read whatever follows - the next window stage or, after the last
  // one, the filter slabs (always more bytes than the overhang). No shared memory is set aside for them.
  s->slack_bytes = 0;
  const int budget = 232448 - 1024 - 1024 - s->slack_bytes;
  for (s->G = 2; s->G >= 1; --s->G) {
    if (planes * s->G * c.Kout > 256 || (s->G > 1 && c.P <= s->R)) continue;   // f32 keeps two accumulators per sub-tile
    s->rows_box = s->G * s->R + (c.Y - 1) * c.dil_h;
    if (s->rows_box > 256) continue;
    s->win_bytes = (s->Wp * s->rows_box + 7) / 8 * 8 * 128;
    // two window stages and at least three slabs; whatever is left goes to more slabs, then a third window stage
    s->wstages = 2;
    const int left = budget - s->wstages * planes * s->win_bytes;
    s->bstages = std::min(kStMaxB, left / (planes * s->slab_bytes));
    if (s->bstages < 3) continue;
    if (s->bstages >= 6 && left - 4 * planes * s->slab_bytes >= planes * s->win_bytes) {
      s->wstages = 3;
      s->bstages = std::min(kStMaxB, (left - planes * s->win_bytes) / (planes * s->slab_bytes));
    }
    return true;
  }
  return false;
}

}  // namespace

bool conv_halo_stream_applicable(const HaloConv& c, int elem_bytes, long long o_k) {
  // f32: the whole reduction of a pixel is ONE accumulation chain in TMEM, and the tensor core adds with truncation (a
  // bias that grows with the chain, csrc/gemm_sm100.cu choose_config). Chains stay at 1024 elements here, half of
  // what the GEMM kernel allows itself, since this kernel cannot cut a chain into K ranges.
  if (elem_bytes == 4 && (long long)c.Y * c.X * c.C > 1024) return false;
  StreamShape s;
  return stream_shape(c, elem_bytes, o_k, &s);
}

RbStatus conv_halo_stream_run(const HaloConv& c, int elem_bytes, const void* image_hi, const void* image_lo, const void* filter_hi,
                              const void* filter_lo, void* out, long long o_k, void* stream_v) {
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  StreamShape s;
  if (!stream_shape(c, elem_bytes, o_k, &s)) return fail(RB_UNSUPPORTED, "convolution outside the reach of the streamed halo kernel");
  const bool f32 = elem_bytes == 4;
  if (f32 && (!image_lo || !filter_lo)) return fail(RB_INVALID_PARAM, "the f32 form needs both TF32 planes of image and filter");
  StreamParams p;
  memset(&p, 0, sizeof(p));
  p.N = c.N; p.P = c.P; p.Q = c.Q; p.Kout = c.Kout; p.cchunks = s.cchunks; p.epr = s.epr;
  p.Y = c.Y; p.X = c.X; p.dil_h = c.dil_h; p.dil_w = c.dil_w; p.pad_h = c.pad_h; p.pad_w = c.pad_w;
  p.Wp = s.Wp; p.R = s.R; p.rows_box = s.rows_box; p.G = s.G;
  p.tiles_per_img = (c.P + s.G * s.R - 1) / (s.G * s.R);
  p.num_tiles = c.N * p.tiles_per_img;
  p.planes = f32 ? 2 : 1;
  p.win_bytes = s.win_bytes; p.wstages = s.wstages; p.slab_bytes = s.slab_bytes; p.bstages = s.bstages; p.slack_bytes = s.slack_bytes;
  const uint32_t fmt = f32 ? 2u : (c.is_bf16 ? 1u : 0u);
  p.idesc = make_idesc(1, fmt, fmt, 0, 0, 128, (uint32_t)c.Kout);
  p.is_bf16 = c.is_bf16;
  p.out = out;
  p.o_n = c.o_n; p.o_p = c.o_p; p.o_q = c.o_q; p.o_k = o_k;
  p.status = dev->status_word;
  p.wait_cycles = kWaitCycles;

  StreamMaps maps;
  memset(&maps, 0, sizeof(maps));
  std::string err;
  const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : (c.is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const void* imgs[2] = {image_hi, image_lo};
  const void* fils[2] = {filter_hi, filter_lo};
  for (int pl = 0; pl < p.planes; ++pl) {
    {
      const uint64_t dims[4] = {(uint64_t)c.C, (uint64_t)c.W, (uint64_t)c.H, (uint64_t)c.N};
      const uint64_t strides[3] = {(uint64_t)c.C * elem_bytes, (uint64_t)c.W * c.C * elem_bytes, (uint64_t)c.H * c.W * c.C * elem_bytes};
      const uint32_t box[4] = {(uint32_t)s.epr, (uint32_t)s.Wp, (uint32_t)s.rows_box, 1u};
      if (!encode_tiled(&maps.in[pl], dt, 4, imgs[pl], dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
        return fail(RB_UNSUPPORTED, "streamed halo kernel, image: " + err);
    }
    {
      const uint64_t ktot = (uint64_t)c.Y * c.X * c.C;
      const uint64_t dims[3] = {ktot, (uint64_t)c.Kout, 1};
      const uint64_t strides[2] = {ktot * elem_bytes, ktot * c.Kout * elem_bytes};
      const uint32_t box[3] = {(uint32_t)s.epr, (uint32_t)c.Kout, 1u};
      if (!encode_tiled(&maps.fil[pl], dt, 3, fils[pl], dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, &err))
        return fail(RB_UNSUPPORTED, "streamed halo kernel, filter: " + err);
    }
  }
  const int smem = s.wstages * p.planes * s.win_bytes + s.slack_bytes + s.bstages * p.planes * s.slab_bytes + 1024 + 1024;
  const void* kern = f32 ? reinterpret_cast<const void*>(conv_halo_stream_kernel<true>) : reinterpret_cast<const void*>(conv_halo_stream_kernel<false>);
  RbStatus st = ensure_dynamic_smem(kern, smem);
  if (st != RB_SUCCESS) return st;
  const int grid = std::min(p.num_tiles, dev->sm_count);
  p.trace = trace_buffer((size_t)grid * 16);
  if (f32) conv_halo_stream_kernel<true><<<grid, kStThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(maps, p);
  else conv_halo_stream_kernel<false><<<grid, kStThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(maps, p);
  RB_CUDA_TRY(cudaGetLastError());
  count_launch();
  return RB_SUCCESS;
}

}  // namespace rb
