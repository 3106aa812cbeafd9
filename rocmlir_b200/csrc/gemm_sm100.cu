// Host side of rbGemm: validates a rock.gemm problem, prepares operands that TMA cannot address
// directly (row pitch not a multiple of 16 bytes -> padded copy in the caller's workspace; f32 ->
// TF32 hi/lo split), encodes the tensor maps and launches the persistent tcgen05 kernel.
#include "gemm_sm100.cuh"

#include <atomic>
#include <cstdio>
#include <mutex>

#include "lib_state.h"

namespace rb {
namespace {

thread_local int t_variant = 0;
thread_local long long t_wait_cycles = kWaitCycles;   // rbSetWaitLimit
thread_local int t_stall_launches = 0;                // rbInjectStall: GEMM launches left to stall
// Chained pair (rbGemmGemm with equal inner extents): the G = 2 problem handed to gemm_run has group 0 = (a, b, c) and
// group 1 = (c of group 0, b2, c2); gemm_run builds tensor maps whose group stride is the distance between the two
// tensors and lets the kernel order the groups through flags (GemmParams::chain_flags).
struct GemmChain {
  const void* b2;
  void* c2;
  unsigned int* flags;
  size_t flags_bytes;
};
thread_local const GemmChain* t_chain = nullptr;

// ---- auxiliary kernels ---------------------------------------------------------------------------
// Copies `rows` rows of `row_bytes` bytes into rows of `pitch_bytes` bytes, zero-filling the pad.
__global__ void pad_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long rows,
                                int row_bytes, int pitch_bytes) {
  const long long total = rows * pitch_bytes;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / pitch_bytes;
    const int c = (int)(i - r * pitch_bytes);
    dst[i] = c < row_bytes ? src[r * row_bytes + c] : (uint8_t)0;
  }
}

// f32 operands are re-laid into K-major planes in the workspace before the TF32 MMA: an MN-major
// operand is transposed (the 32-bit MN-major shared-memory layout needs a different swizzle mode, so
// the kernel keeps a single K-major path for TF32), rows are pitched to a multiple of 16 bytes, and with
// SPLIT the value is separated into x = hi + lo (+ O(2^-22 |x|)) with hi and lo both exactly
// representable in TF32 (low 13 mantissa bits zero), so that hi*hi + hi*lo + lo*hi carries fp32-class
// accuracy whatever the tensor core does with the low bits.
//   src: [G][R][C] row-major.  TRANSPOSE = false: out [G][R][pitch] (pitch >= C)
//                              TRANSPOSE = true : out [G][C][pitch] (pitch >= R)
__device__ __forceinline__ float tf32_round(float x) {
  const uint32_t xb = __float_as_uint(x);
  if ((xb & 0x7F800000u) == 0x7F800000u) return x;  // inf / nan
  return __uint_as_float((xb + 0x1000u) & 0xFFFFE000u);
}
template <bool TRANSPOSE, bool SPLIT>
__global__ void f32_prepare_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo,
                                   int R, int C, int pitch, int tiles_x, int tiles_y, long long total_tiles) {
  __shared__ float tile[32][33];
  // 32 x 32 tiles dealt out over a 1-D grid: row counts of several million (im2col matrices) exceed gridDim.y
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const long long g = t / ((long long)tiles_x * tiles_y);
    const long long rem = t - g * (long long)tiles_x * tiles_y;
    const int c0 = (int)(rem % tiles_x) * 32, r0 = (int)(rem / tiles_x) * 32;
    const float* s = src + g * (long long)R * C;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + threadIdx.y + 8 * i, c = c0 + threadIdx.x;
      tile[threadIdx.y + 8 * i][threadIdx.x] = (r < R && c < C) ? s[(long long)r * C + c] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float x;
      long long o;
      bool ok;
      if (TRANSPOSE) {
        const int oc = c0 + threadIdx.y + 8 * i;  // output row = source column
        const int orr = r0 + threadIdx.x;         // output column = source row
        x = tile[threadIdx.x][threadIdx.y + 8 * i];
        ok = oc < C && orr < pitch;
        o = (g * C + oc) * (long long)pitch + orr;
      } else {
        const int r = r0 + threadIdx.y + 8 * i, c = c0 + threadIdx.x;
        x = tile[threadIdx.y + 8 * i][threadIdx.x];
        ok = r < R && c < pitch;
        o = (g * R + r) * (long long)pitch + c;
      }
      if (ok) {
        if (SPLIT) {
          const float h = tf32_round(x);
          const float l = isfinite(h) ? tf32_round(x - h) : 0.0f;
          hi[o] = h;
          lo[o] = l;
        } else {
          hi[o] = x;
        }
      }
    }
    __syncthreads();
  }
}

// ---- dispatch ----------------------------------------------------------------------------------------
typedef void (*GemmKernel)(const GemmTensorMaps, const GemmParams);

template <int KIND, int CTAS, bool EPI>
GemmKernel pick_major(bool a_mn, bool b_mn) {
  if (!a_mn && !b_mn) return gemm_tcgen05_kernel<KIND, false, false, CTAS, EPI>;
  if (!a_mn && b_mn) return gemm_tcgen05_kernel<KIND, false, true, CTAS, EPI>;
  if (a_mn && !b_mn) return gemm_tcgen05_kernel<KIND, true, false, CTAS, EPI>;
  return gemm_tcgen05_kernel<KIND, true, true, CTAS, EPI>;
}
template <int CTAS, bool EPI>
GemmKernel pick_kernel(int kind, bool a_mn, bool b_mn) {
  switch (kind) {
    case kKindF16: return pick_major<kKindF16, CTAS, EPI>(a_mn, b_mn);
    case kKindTF32: return gemm_tcgen05_kernel<kKindTF32, false, false, CTAS, EPI>;  // f32 operands are made K-major first
    case kKindI8: return pick_major<kKindI8, CTAS, EPI>(a_mn, b_mn);
    default: return pick_major<kKindF8, CTAS, EPI>(a_mn, b_mn);
  }
}

// ---- tile configuration -----------------------------------------------------------------------
// The measured tile-shape table of this library, in the role of rocMLIR's perf_config heuristics
// (mlir/lib/Dialect/Rock/Tuning/GridwiseGemmParams.cpp:384-417): tile width from N, CTA pairs whenever
// the operand layout allows them, the deepest ring that fits, and a K split when the output has too few
// tiles to fill the GPU (the role of split-K in mlir/lib/Dialect/Rock/Transforms/GemmToGridwise.cpp:268-394,
// here with f32 partial planes and a fixed-order reduction instead of atomics).
// Planning uses the SM count of the current device when one is present (148 on a B200) and 148 otherwise, so that
// the configuration queries answer the same on a build machine without a GPU.
int planned_sms() { return planning_sm_count(); }

struct GemmConfig {
  int ctas, bn, stages, splits;
  int kpr;                 // K blocks per barrier round (see GemmParams::kpr)
  bool plain_stores;
  int dp_tiles, sk_tiles;  // stream-K tail (see GemmParams); sk_tiles == 0: every tile is computed whole
};

GemmConfig choose_config(const RbGemmProblem* p, int variant, bool epi_vec = false) {
  GemmConfig c;
  if (variant == 0) variant = (int)tuned_variant_gemm(p);   // the measured table, when it knows the problem
  const int es = (int)dtype_bytes(p->ab_type);
  const bool b_mn = p->ab_type != RB_F32 && p->trans_b == 0;
  const int che = kRowBytes / es;
  const int bn_code = (variant >> 12) & 0xF;
  c.bn = bn_code == 1 ? 64 : bn_code == 2 ? 128 : bn_code == 3 ? 256 : (p->n <= 64 ? 64 : p->n <= 128 ? 128 : 256);
  if (b_mn && c.bn < che) c.bn = che;                       // an MN-major B tile is loaded in whole 128-byte chunks
  c.ctas = ((variant & 0xF) == 1) ? 1 : 2;
  if (b_mn && (c.bn / 2) % che != 0) c.ctas = 1;
  if (p->m <= kBM && (variant & 0xF) != 2) c.ctas = 1;      // a pair would compute 128 empty rows
  {
    // a main loop of one or two K blocks leaves the epilogue exposed, and the epilogue of a pair is the slower one
    // (measured at K = 64, 256 columns: 134 us paired, 86 us unpaired, the HBM floor being 79 us)
    const long long kb = (p->k + kRowBytes / es - 1) / (kRowBytes / es);
    if (kb <= 2 && (variant & 0xF) != 2) c.ctas = 1;
  }
  if (c.bn == 64 && (variant & 0xF) != 2) c.ctas = 1;        // measured: 64-column tiles run faster unpaired (345 vs 324 TFLOP/s)
  c.stages = (variant >> 4) & 0xF;
  const int max_stages = c.ctas == 2 ? GemmSmemLayout<2>::max_stages(c.bn, epi_vec) : GemmSmemLayout<1>::max_stages(c.bn, epi_vec);
  if (c.stages <= 0 || c.stages > max_stages) c.stages = max_stages;
  // K blocks per barrier round. One round costs the issuing thread about 310 + 44 n cycles for n MMAs (measured),
  // which four 128x256x16 MMAs (512 cycles) barely hide and four narrower ones do not. Measured: two blocks per
  // round at 256 columns (4096^3 f16 1100 -> 1290 TFLOP/s with this producer loop), four at 128 and 64 columns.
  // Variant bits 28-29: 1, 2, 3 = 1, 2, 4 blocks; 0 = this rule.
  const int kpr_code = (variant >> 28) & 3;
  c.kpr = kpr_code == 1 ? 1 : kpr_code == 2 ? 2 : kpr_code == 3 ? 4 : (c.bn <= 128 ? 4 : 2);
  while (c.kpr > 1 && c.stages < 2 * c.kpr) c.kpr /= 2;   // at least two rounds in flight
  c.stages = c.stages / c.kpr * c.kpr;
  c.plain_stores = ((variant >> 8) & 1) != 0;
  const int bke = kRowBytes / es;
  const long long kblocks = (p->k + bke - 1) / bke;
  const long long tiles = (long long)p->g * ((p->m + kBM * c.ctas - 1) / (kBM * c.ctas)) * ((p->n + c.bn - 1) / c.bn);
  const long long units = planned_sms() / c.ctas;
  c.splits = (variant >> 16) & 0xFF;
  if (c.splits == 0) {
    c.splits = 1;
    if (tiles * 2 <= units && kblocks >= 16) {
      long long want = units / tiles;
      long long cap = kblocks / 8;  // at least 8 K blocks per range
      c.splits = (int)std::max<long long>(1, std::min<long long>(std::min(want, cap), 128));
    }
  }
  // f32 in accurate mode: the tensor core adds each MMA's products into the f32 accumulator with truncation, a bias
  // of about -2^-24 per 8-element step that grows linearly with the length of one accumulation chain (measured:
  // relative error 7.5e-9 x K on same-sign data; 1.9e-4 at K = 25088, where the sequential f32 loop of the reference
  // has 1e-5). Chains are therefore kept to 2048 elements; the partial planes are added with round-to-nearest.
  if (p->ab_type == RB_F32 && p->f32_mode == 0) {   // also under an explicit variant: shorter chains only
    const long long need = std::min<long long>(((long long)p->k + 2047) / 2048, 255);
    if (need > c.splits) c.splits = (int)need;
  }
  if (c.splits > kblocks) c.splits = (int)kblocks;
  // every range must be non-empty with ceil-division ranges
  while (c.splits > 1 && (long long)(c.splits - 1) * ((kblocks + c.splits - 1) / c.splits) >= kblocks) --c.splits;
  // Stream-K tail (variant bit 9 switches it ON): when the last wave of whole tiles would leave more than 5 % of the
  // GPU idle, the tiles of the last full wave plus the remainder are dealt out by K blocks instead. Measured on
  // B200 it does not pay for the shapes tried (4096^3 f16: 1090 vs 1120 TFLOP/s sustained; 2048x11008x4096 i8:
  // 2000 vs 2300 TOP/s): the GPU runs at its power cap, idle SMs in the last wave let the busy ones clock higher,
  // and the short partial items expose their epilogues. It stays available for tuning.
  c.dp_tiles = (int)tiles;
  c.sk_tiles = 0;
  if (c.splits == 1 && tiles > units && ((variant >> 9) & 1) && kblocks >= 8) {
    const long long rem = tiles % units;
    const long long waves = (tiles + units - 1) / units;
    if (rem != 0 && (double)(units - rem) / (double)(waves * units) > 0.05) {
      c.sk_tiles = (int)(rem + units);
      c.dp_tiles = (int)(tiles - c.sk_tiles);
    }
  }
  return c;
}

// Sums the partial planes of a K split in a fixed order (range 0, 1, 2, ...), applies the epilogue and
// writes C. One thread per output element; consecutive threads walk consecutive columns.
__global__ void splitk_reduce_kernel(const void* __restrict__ partial, int splits, long long plane, int G, int M, int N,
                                     void* __restrict__ c, int c_type, int trans_c, int acc_is_int, EpiParams epi) {
  const long long total = (long long)G * M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i % N);
    const long long gm = i / N;
    const int m = (int)(gm % M);
    const long long g = gm / M;
    const long long o = trans_c ? (g * N + n) * (long long)M + m : i;
    if (acc_is_int) {
      int acc = 0;
      for (int s = 0; s < splits; ++s) acc += reinterpret_cast<const int*>(partial)[s * plane + i];
      if (c_type == RB_I32 && epi.flags == 0) {
        reinterpret_cast<int*>(c)[o] = acc;
      } else {
        float x = __int2float_rn(acc);
        if (epi.flags) x = epi_apply(x, epi, n, m, o);
        store_elem(c, o, x, c_type, epi.out_zero);
      }
    } else {
      float acc = 0.0f;
      for (int s = 0; s < splits; ++s) acc = __fadd_rn(acc, reinterpret_cast<const float*>(partial)[s * plane + i]);
      if (epi.flags) acc = epi_apply(acc, epi, n, m, o);
      store_elem(c, o, acc, c_type, epi.out_zero);
    }
  }
}

struct OperandPlan {
  bool src_mn_major;    // as stored by the caller: contiguous dimension is M/N (not K)
  bool mn_major;        // as the kernel sees it (after a transposing copy, if any)
  int src_rows, src_cols;  // stored matrix per batch
  long long rows;       // rows per batch as the kernel sees it
  int cols;             // contiguous extent as the kernel sees it
  int pitch;            // elements per row as the kernel sees it
  bool needs_copy;      // operand goes through the workspace
};

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

OperandPlan plan_operand(bool mn_major, int mn, int k, size_t es, bool is_f32, bool split) {
  OperandPlan o;
  o.src_mn_major = mn_major;
  o.src_rows = mn_major ? k : mn;
  o.src_cols = mn_major ? mn : k;
  o.mn_major = is_f32 ? false : mn_major;
  o.rows = o.mn_major ? k : mn;
  o.cols = o.mn_major ? mn : k;
  const int elems16 = (int)(16 / es);
  o.pitch = (o.cols + elems16 - 1) / elems16 * elems16;
  o.needs_copy = o.pitch != o.cols || (is_f32 && (split || mn_major));
  return o;
}

bool valid_ab(int t) {
  return t == RB_F32 || t == RB_F16 || t == RB_BF16 || t == RB_I8 || (t >= RB_F8E4M3 && t <= RB_F8E5M2_E4M3);
}
bool valid_c(int t) { return t >= RB_F32 && t <= RB_F8E4M3; }

RbStatus check_problem(const RbGemmProblem* p) {
  if (!p) return fail(RB_INVALID_PARAM, "problem is NULL");
  if (p->g <= 0 || p->m <= 0 || p->n <= 0 || p->k <= 0) return fail(RB_INVALID_PARAM, "g, m, n, k must be positive");
  if (!valid_ab(p->ab_type) || !valid_c(p->c_type)) return fail(RB_INVALID_PARAM, "unknown element type");
  return RB_SUCCESS;
}

struct Workspace {
  size_t a_off[2], b_off[2];  // [0] = copy / hi, [1] = lo
  size_t partial_off;         // K-split partial planes
  size_t sk_off, sk_flags_off;  // stream-K partial tiles and their arrival counters
  size_t total;
};

Workspace plan_workspace(const RbGemmProblem* p, const OperandPlan& oa, const OperandPlan& ob, const GemmConfig& cfg) {
  Workspace w{};
  const size_t es = dtype_bytes(p->ab_type);
  const bool split = p->ab_type == RB_F32 && p->f32_mode == 0;
  size_t off = 0;
  const size_t a_bytes = align_up((size_t)p->g * oa.rows * oa.pitch * es, 256);
  const size_t b_bytes = align_up((size_t)p->g * ob.rows * ob.pitch * es, 256);
  if (oa.needs_copy) { w.a_off[0] = off; off += a_bytes; }
  if (split && oa.needs_copy) { w.a_off[1] = off; off += a_bytes; }
  if (ob.needs_copy) { w.b_off[0] = off; off += b_bytes; }
  if (split && ob.needs_copy) { w.b_off[1] = off; off += b_bytes; }
  if (cfg.splits > 1) {
    w.partial_off = off;
    off += align_up((size_t)cfg.splits * p->g * p->m * p->n * 4, 256);
  }
  if (cfg.sk_tiles > 0) {
    const size_t units = planned_sms() / cfg.ctas;
    w.sk_off = off;
    off += align_up(units * (size_t)(kBM * cfg.ctas) * cfg.bn * 4, 256);
    w.sk_flags_off = off;
    off += align_up(units * 8 * sizeof(unsigned int), 256);
  }
  w.total = off;
  return w;
}


}  // namespace
}  // namespace rb

using namespace rb;

extern "C" void rbSetGemmVariant(int variant) { t_variant = variant; }
extern "C" int rbGetGemmVariant(void) { return t_variant; }
extern "C" void rbSetWaitLimit(uint64_t sm_cycles) {
  t_wait_cycles = sm_cycles == 0 ? kWaitCycles : (long long)std::min<uint64_t>(sm_cycles, (uint64_t)1 << 40);
}
extern "C" void rbInjectStall(int launches) { t_stall_launches = launches > 0 ? launches : 0; }

size_t rb::gemm_workspace_bytes(const RbGemmProblem* p, int implicit_operand) {
  if (check_problem(p) != RB_SUCCESS) return 0;
  const size_t es = dtype_bytes(p->ab_type);
  const bool f32 = p->ab_type == RB_F32, split = f32 && p->f32_mode == 0;
  OperandPlan oa = plan_operand(p->trans_a != 0, p->m, p->k, es, f32, split);
  OperandPlan ob = plan_operand(p->trans_b == 0, p->n, p->k, es, f32, split);
  if (implicit_operand == 0) oa.needs_copy = false;
  if (implicit_operand == 1) ob.needs_copy = false;
  return plan_workspace(p, oa, ob, choose_config(p, t_variant)).total;
}

extern "C" size_t rbGemmWorkspaceSize(const RbGemmProblem* p) { return rb::gemm_workspace_bytes(p, -1); }

RbStatus rb::f32_planes(const float* src, float* hi, float* lo, int groups, int R, int C, int pitch, bool transpose,
                        bool split, void* stream_v) {
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const dim3 blk(32, 8, 1);
  const int cx = transpose ? C : pitch, ry = transpose ? pitch : R;
  const int tiles_x = (cx + 31) / 32, tiles_y = (ry + 31) / 32;
  const long long total_tiles = (long long)tiles_x * tiles_y * groups;
  const dim3 grd((unsigned)std::min<long long>(total_tiles, (long long)dev->sm_count * 64), 1, 1);
  if (transpose) {
    if (split) f32_prepare_kernel<true, true><<<grd, blk, 0, stream>>>(src, hi, lo, R, C, pitch, tiles_x, tiles_y, total_tiles);
    else f32_prepare_kernel<true, false><<<grd, blk, 0, stream>>>(src, hi, lo, R, C, pitch, tiles_x, tiles_y, total_tiles);
  } else {
    if (split) f32_prepare_kernel<false, true><<<grd, blk, 0, stream>>>(src, hi, lo, R, C, pitch, tiles_x, tiles_y, total_tiles);
    else f32_prepare_kernel<false, false><<<grd, blk, 0, stream>>>(src, hi, lo, R, C, pitch, tiles_x, tiles_y, total_tiles);
  }
  count_launch();
  RB_CUDA_TRY(cudaGetLastError());
  return RB_SUCCESS;
}

extern "C" RbStatus rbGemmGetConfig(const RbGemmProblem* p, RbGemmConfigInfo* out) {
  RbStatus st = check_problem(p);
  if (st != RB_SUCCESS) return st;
  if (!out) return fail(RB_INVALID_PARAM, "out is NULL");
  const GemmConfig c = choose_config(p, t_variant);
  const int es = (int)dtype_bytes(p->ab_type);
  const long long tiles = (long long)p->g * ((p->m + kBM * c.ctas - 1) / (kBM * c.ctas)) * ((p->n + c.bn - 1) / c.bn);
  const long long items = tiles * c.splits;
  const long long units = planned_sms() / c.ctas;
  memset(out, 0, sizeof(*out));
  out->tile_m = kBM * c.ctas;
  out->tile_n = c.bn;
  out->tile_k = kRowBytes / es;
  out->ctas = c.ctas;
  out->stages = c.stages;
  out->splits = c.splits;
  out->stream_k = c.sk_tiles > 0 ? 1 : 0;
  out->grid = (uint32_t)(c.ctas * std::min<long long>(items, units));
  out->block = kGemmThreads;
  out->dynamic_smem = (uint32_t)(c.ctas == 2 ? GemmSmemLayout<2>::total(c.stages, c.bn, false)
                                              : GemmSmemLayout<1>::total(c.stages, c.bn, false));
  // with per-column epilogue vectors (bias / column scales) the ring may be one stage shorter and the staging single
  {
    const GemmConfig ce = choose_config(p, t_variant, true);
    out->stages_epi_vec = ce.stages;
    out->dynamic_smem_epi_vec = (uint32_t)(ce.ctas == 2 ? GemmSmemLayout<2>::total(ce.stages, ce.bn, true)
                                                        : GemmSmemLayout<1>::total(ce.stages, ce.bn, true));
  }
  out->kpr = c.kpr;
  const int bn_code = c.bn == 64 ? 1 : c.bn == 128 ? 2 : 3;
  const int kpr_code = c.kpr == 1 ? 1 : c.kpr == 2 ? 2 : 3;
  out->variant = (uint32_t)c.ctas | ((uint32_t)c.stages << 4) | (c.plain_stores ? 1u << 8 : 0u) |
                 (c.sk_tiles > 0 ? 1u << 9 : 0u) | ((uint32_t)bn_code << 12) | ((uint32_t)c.splits << 16) |
                 ((uint32_t)kpr_code << 28);
  return RB_SUCCESS;
}

extern "C" RbStatus rbGemm(const RbGemmProblem* p, const RbEpilogue* epi, const void* a, const void* b, void* c,
                           void* workspace, size_t workspace_bytes, void* stream_v) {
  return rb::gemm_run(p, epi, a, b, c, workspace, workspace_bytes, stream_v, nullptr);
}

// Name of an instantiation of gemm_tcgen05_kernel inside the cubin image (Itanium mangling of
// rb::gemm_tcgen05_kernel<KIND, A_MN, B_MN, CTAS, EPI>(GemmTensorMaps, GemmParams)).
static std::string kernel_symbol(int kind, bool a_mn, bool b_mn, int ctas, bool epi) {
  return "_ZN2rb19gemm_tcgen05_kernelILi" + std::to_string(kind) + "ELb" + (a_mn ? "1" : "0") + "ELb" + (b_mn ? "1" : "0") +
         "ELi" + std::to_string(ctas) + "ELb" + (epi ? "1" : "0") + "EEEvNS_14GemmTensorMapsENS_10GemmParamsE";
}

RbStatus rb::gemm_run(const RbGemmProblem* p, const RbEpilogue* epi, const void* a, const void* b, void* c,
                      void* workspace, size_t workspace_bytes, void* stream_v, const ConvAOperand* conva,
                      RbKernelLaunch* capture) {
  RbStatus st = check_problem(p);
  if (st != RB_SUCCESS) return st;
  const bool conv_a = conva && conva->operand == 0, conv_b = conva && conva->operand == 1;
  if (conva) {
    const bool f32_ok = conv_a && (p->f32_mode != 0 || conva->tensor_lo);   // TF32 planes prepared by the caller
    if (p->g != 1 || (conv_a && p->trans_a) || (conv_b && p->trans_b) || (p->ab_type == RB_F32 && !f32_ok) || !conva->tensor)
      return fail(RB_UNSUPPORTED, "implicit operand: one group, A K-major or B stored K x N (f32: A only, as TF32 planes)");
    if (conv_a) a = conva->tensor;
    else b = conva->tensor;
  }
  if (!a || !b || !c) return fail(RB_INVALID_PARAM, "a, b and c must be device pointers");
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const int abt = p->ab_type;
  const size_t es = dtype_bytes(abt);
  const bool is_int = abt == RB_I8;
  const uint32_t flags = (epi ? epi->flags : 0u) | (p->store_method == 1 ? (uint32_t)RB_EPI_RESIDUAL : 0u);
  if (is_int && flags == 0 && p->c_type != RB_I32)
    return fail(RB_UNSUPPORTED, "i8 x i8 without an epilogue produces i32 (rocmlir-gen: -t i8 implies an i32 result)");
  if (!is_int && p->c_type == RB_I32) return fail(RB_UNSUPPORTED, "float inputs cannot produce an i32 result");
  if (p->store_method != 0 && p->store_method != 1) return fail(RB_INVALID_PARAM, "store_method must be 0 (set) or 1 (add)");
  if (p->store_method == 1) {
    // C += A.B (rock.gemm with store_method = atomic_add, RockOps.td:136-181): the fused residual step reading C itself
    if (!(p->c_type == RB_F32 || p->c_type == RB_F16 || p->c_type == RB_BF16))
      return fail(RB_UNSUPPORTED, "store_method add exists for f32, f16 and bf16 results");
    if (epi && (epi->flags & RB_EPI_RESIDUAL)) return fail(RB_UNSUPPORTED, "store_method add cannot be combined with a residual operand");
  }
  if (epi) {
    if ((flags & RB_EPI_COL_SCALE) && !epi->col_scale) return fail(RB_INVALID_PARAM, "col_scale is NULL");
    if ((flags & RB_EPI_BIAS) && !epi->bias) return fail(RB_INVALID_PARAM, "bias is NULL");
    if ((flags & RB_EPI_BIAS) && !(epi->bias_type == RB_F32 || epi->bias_type == RB_F16 || epi->bias_type == RB_BF16))
      return fail(RB_INVALID_PARAM, "bias_type must be f32, f16 or bf16");
    if ((flags & RB_EPI_BIAS_ROW) && (flags & RB_EPI_BIAS_SCALAR)) return fail(RB_INVALID_PARAM, "bias is per row or scalar, not both");
    if ((epi->flags & RB_EPI_RESIDUAL) && !epi->residual) return fail(RB_INVALID_PARAM, "residual is NULL");
    if ((epi->flags & RB_EPI_RESIDUAL) && !(epi->res_type == RB_F32 || epi->res_type == RB_F16 || epi->res_type == RB_BF16))
      return fail(RB_INVALID_PARAM, "res_type must be f32, f16 or bf16");
    if ((epi->flags & RB_EPI_UNARY) && (epi->unary <= RB_UNARY_NONE || epi->unary > RB_UNARY_TANH))
      return fail(RB_INVALID_PARAM, "unary must name one of the RbUnary functions");
    if ((flags & RB_EPI_CLIP) && !(epi->clip_lo <= epi->clip_hi)) return fail(RB_INVALID_PARAM, "clip needs lo <= hi");
    if ((flags & RB_EPI_ZP_OUT) && p->c_type != RB_I8) return fail(RB_INVALID_PARAM, "an output zero point needs an i8 result");
  }

  int kind;
  uint32_t fmt, fmt_b = 0xffffffffu, cfmt = 1;   // fmt_b: B's format when it differs from A's
  switch (abt) {
    case RB_F16: kind = kKindF16; fmt = 0; break;
    case RB_BF16: kind = kKindF16; fmt = 1; break;
    case RB_F32: kind = kKindTF32; fmt = 2; break;
    case RB_I8: kind = kKindI8; fmt = 1; cfmt = 2; break;
    case RB_F8E5M2: kind = kKindF8; fmt = 1; break;               // f8f6f4 kind: 0 = e4m3, 1 = e5m2
    case RB_F8E4M3_E5M2: kind = kKindF8; fmt = 0; fmt_b = 1; break;
    case RB_F8E5M2_E4M3: kind = kKindF8; fmt = 1; fmt_b = 0; break;
    default: kind = kKindF8; fmt = 0; break;
  }

  const bool is_f32 = abt == RB_F32;
  const bool split = is_f32 && p->f32_mode == 0;
  OperandPlan oa = plan_operand(p->trans_a != 0 /* A stored G x K x M */, p->m, p->k, es, is_f32, split);
  if (conv_a) {  // fetched in place by im2col loads: never copied, never padded
    oa.needs_copy = false;
    oa.pitch = oa.cols;
  }
  OperandPlan ob = plan_operand(p->trans_b == 0 /* B stored G x K x N */, p->n, p->k, es, is_f32, split);
  if (conv_b) {
    ob.needs_copy = false;
    ob.pitch = ob.cols;
  }
  const bool a_mn = oa.mn_major, b_mn = ob.mn_major;
  const bool epi_vec = epi_needs_col_vectors(flags);
  GemmConfig cfg = choose_config(p, t_variant, epi_vec);
  Workspace ws = plan_workspace(p, oa, ob, cfg);
  if (cfg.sk_tiles > 0 && (!workspace || workspace_bytes < ws.total)) {
    // the stream-K tail is an optimisation: without room for its partial tiles every tile is computed whole
    cfg.sk_tiles = 0;
    ws = plan_workspace(p, oa, ob, cfg);
  }
  const GemmChain* chain = t_chain;
  // group 1 of a chained pair: A is group 0's C, B and C are the chain's; base = lower address, stride = distance
  const void* chain_ptr[3][2] = {{a, c}, {b, chain ? chain->b2 : nullptr}, {c, chain ? chain->c2 : nullptr}};
  uint64_t chain_stride[3] = {0, 0, 0};
  int chain_flip = 0;
  if (chain) {
    if (p->g != 2 || oa.needs_copy || ob.needs_copy || cfg.splits != 1 || conva || epi || capture || p->trans_c ||
        p->store_method != 0 || p->c_type != abt || p->k != p->n)
      return fail(RB_UNSUPPORTED, "this pair of products does not run as one chained launch");
    if (cfg.sk_tiles > 0) { cfg.sk_tiles = 0; ws = plan_workspace(p, oa, ob, cfg); }
    for (int i = 0; i < 3; ++i) {
      const uintptr_t x0 = reinterpret_cast<uintptr_t>(chain_ptr[i][0]), x1 = reinterpret_cast<uintptr_t>(chain_ptr[i][1]);
      const uintptr_t d = x1 > x0 ? x1 - x0 : x0 - x1;
      if (d == 0 || d % 16 || x0 % 16 || d >= ((uintptr_t)1 << 40))
        return fail(RB_UNSUPPORTED, "chained launch: the two tensors of an operand must be distinct, 16-byte aligned and within 2^40 bytes");
      chain_stride[i] = (uint64_t)d;
      if (x1 < x0) chain_flip |= 1 << i;
    }
  }
  if (capture && (oa.needs_copy || ob.needs_copy || cfg.splits > 1))
    return fail(RB_UNSUPPORTED, "this problem runs as several kernels (operand copy, TF32 planes or a K split): it has no "
                                "single-kernel binary; launch it through the library");
  if (ws.total > 0) {
    if (!workspace || workspace_bytes < ws.total)
      return fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(ws.total) + " bytes required");
    if (reinterpret_cast<uintptr_t>(workspace) % 16) return fail(RB_INVALID_PARAM, "workspace must be 16-byte aligned");
  }
  if ((reinterpret_cast<uintptr_t>(a) % 16 && !oa.needs_copy) || (reinterpret_cast<uintptr_t>(b) % 16 && !ob.needs_copy))
    return fail(RB_UNSUPPORTED, "operand base addresses must be 16-byte aligned");

  uint8_t* wsb = static_cast<uint8_t*>(workspace);
  const void* a_src[2] = {a, nullptr};
  const void* b_src[2] = {b, nullptr};
  auto prepare_f32 = [&](const void* src, const OperandPlan& o, float* hi, float* lo) {
    const dim3 blk(32, 8, 1);
    // the grid covers the padded extent of whichever dimension becomes the output row pitch
    const int cx = o.src_mn_major ? o.src_cols : o.pitch, ry = o.src_mn_major ? o.pitch : o.src_rows;
    const int tiles_x = (cx + 31) / 32, tiles_y = (ry + 31) / 32;
    const long long total_tiles = (long long)tiles_x * tiles_y * p->g;
    const dim3 grd((unsigned)std::min<long long>(total_tiles, (long long)dev->sm_count * 64), 1, 1);
    const float* s = static_cast<const float*>(src);
    if (o.src_mn_major) {
      if (split) f32_prepare_kernel<true, true><<<grd, blk, 0, stream>>>(s, hi, lo, o.src_rows, o.src_cols, o.pitch, tiles_x, tiles_y, total_tiles);
      else f32_prepare_kernel<true, false><<<grd, blk, 0, stream>>>(s, hi, lo, o.src_rows, o.src_cols, o.pitch, tiles_x, tiles_y, total_tiles);
    } else {
      if (split) f32_prepare_kernel<false, true><<<grd, blk, 0, stream>>>(s, hi, lo, o.src_rows, o.src_cols, o.pitch, tiles_x, tiles_y, total_tiles);
      else f32_prepare_kernel<false, false><<<grd, blk, 0, stream>>>(s, hi, lo, o.src_rows, o.src_cols, o.pitch, tiles_x, tiles_y, total_tiles);
    }
    count_launch();
  };
  if (is_f32) {
    if (oa.needs_copy) {
      float* hi = reinterpret_cast<float*>(wsb + ws.a_off[0]);
      float* lo = split ? reinterpret_cast<float*>(wsb + ws.a_off[1]) : nullptr;
      prepare_f32(a, oa, hi, lo);
      a_src[0] = hi; a_src[1] = lo;
    }
    if (ob.needs_copy) {
      float* hi = reinterpret_cast<float*>(wsb + ws.b_off[0]);
      float* lo = split ? reinterpret_cast<float*>(wsb + ws.b_off[1]) : nullptr;
      prepare_f32(b, ob, hi, lo);
      b_src[0] = hi; b_src[1] = lo;
    }
  } else {
    if (oa.needs_copy) {
      pad_rows_kernel<<<dev->sm_count * 4, 256, 0, stream>>>(static_cast<const uint8_t*>(a), wsb + ws.a_off[0],
                                                           (long long)p->g * oa.rows, (int)(oa.cols * es),
                                                           (int)(oa.pitch * es));
      count_launch();
      a_src[0] = wsb + ws.a_off[0];
    }
    if (ob.needs_copy) {
      pad_rows_kernel<<<dev->sm_count * 4, 256, 0, stream>>>(static_cast<const uint8_t*>(b), wsb + ws.b_off[0],
                                                           (long long)p->g * ob.rows, (int)(ob.cols * es),
                                                           (int)(ob.pitch * es));
      count_launch();
      b_src[0] = wsb + ws.b_off[0];
    }
  }
  RB_CUDA_TRY(cudaGetLastError());   // launch errors of the preparation kernels

  // Variant word (rbSetGemmVariant): bits 0-3: 1 = single CTA per tile, 2 = CTA pair (0 = automatic);
  // bits 4-7 ring depth; bit 8 plain stores instead of TMA stores; bits 12-15 tile width code (1 = 64,
  // 2 = 128, 3 = 256); bits 16-23 K-split count. Zero fields mean "choose" (see choose_config).
  const int ctas = cfg.ctas, bn = cfg.bn, stages = cfg.stages, splits = cfg.splits;

  const int bke = (int)(kRowBytes / es);
  GemmTensorMaps maps;
  memset(&maps, 0, sizeof(maps));
  CUtensorMapDataType dt = abt == RB_F16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : abt == RB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : abt == RB_F32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  // An MN-major tile is 128-byte chunks of M/N x K rows; when the extent is a whole number of chunks the chunk
  // index becomes a tensor dimension of its own and one 4-D box fetches the whole tile of a stage.
  const bool a_fused = oa.mn_major && oa.cols % bke == 0 && oa.pitch == oa.cols;
  const bool b_fused = ob.mn_major && ob.cols % bke == 0 && ob.pitch == ob.cols;
  auto encode_operand = [&](CUtensorMap* m, const void* base, const OperandPlan& o, int box_rows_kmajor,
                            std::string* err) {
    const bool fused = (&o == &oa) ? a_fused : b_fused;
    const int ci = (&o == &oa) ? 0 : 1;
    const uint64_t gstride = chain ? chain_stride[ci] : (uint64_t)o.rows * o.pitch * es;
    if (chain) base = (chain_flip >> ci) & 1 ? chain_ptr[ci][1] : chain_ptr[ci][0];
    if (fused) {
      const uint64_t dims[4] = {(uint64_t)bke, (uint64_t)o.rows, (uint64_t)(o.cols / bke), (uint64_t)p->g};
      const uint64_t strides[3] = {(uint64_t)o.pitch * es, (uint64_t)kRowBytes, gstride};
      const uint32_t box[4] = {(uint32_t)bke, (uint32_t)bke, (uint32_t)(box_rows_kmajor / bke), 1u};
      return encode_tiled(m, dt, 4, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
    }
    const uint64_t dims[3] = {(uint64_t)o.cols, (uint64_t)o.rows, (uint64_t)p->g};
    const uint64_t strides[2] = {(uint64_t)o.pitch * es, gstride};
    // K-major: box = BKE k-elements x tile rows. MN-major: box = one 128-byte chunk of MN x BKE k-rows.
    const uint32_t box[3] = {(uint32_t)bke, (uint32_t)(o.mn_major ? bke : box_rows_kmajor), 1u};
    return encode_tiled(m, dt, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
  };
  std::string err;
  // Segment order for the split: (lo,hi), (hi,lo), (hi,hi) so that the small terms are summed first.
  const int nseg = split ? 3 : 1;
  const int seg_a[3] = {split ? 1 : 0, 0, 0};
  const int seg_b[3] = {0, 1, 0};
  if (conva) {
    const ConvAOperand& cv = *conva;
    const int che = kRowBytes / (int)es;   // elements per 128-byte run of channels
    if (cv.C % che != 0) return fail(RB_UNSUPPORTED, "implicit operand: channels must be a multiple of 128 bytes");
    const long long pixels = (long long)cv.N * cv.P * cv.Q, taps = (long long)cv.Y * cv.X * cv.C;
    if (conv_a ? (pixels != p->m || taps != p->k) : (pixels != p->k || taps != p->n))
      return fail(RB_INVALID_PARAM, "implicit operand does not match the GEMM extents");
    const uint64_t dims[4] = {(uint64_t)cv.C, (uint64_t)cv.W, (uint64_t)cv.H, (uint64_t)cv.N};
    const uint64_t strides[3] = {(uint64_t)cv.C * es, (uint64_t)cv.W * cv.C * es, (uint64_t)cv.H * cv.W * cv.C * es};
    // bounding box of the base pixel: from -pad to (extent - 1) + upper corner, so that stepping by the stride
    // visits exactly P x Q positions (CUTLASS states the same rule for its fprop maps)
    const int lower[2] = {-cv.pad_w, -cv.pad_h};
    const int upper[2] = {cv.pad_w_hi - (cv.X - 1) * cv.dil_w, cv.pad_h_hi - (cv.Y - 1) * cv.dil_h};
    const uint32_t trav[2] = {(uint32_t)cv.stride_w, (uint32_t)cv.stride_h};
    // A: a tile is 128 pixels (rows) x one K block of channels. B: a chunk is one K block of pixels x 64 channels.
    for (int sg = 0; sg < (conv_a ? nseg : 1); ++sg) {
      // f32 accurate mode: segment sg of A reads the lo or the hi plane (same order as the copied-operand path)
      const void* plane = (conv_a && seg_a[sg] == 1) ? cv.tensor_lo : cv.tensor;
      if (!encode_im2col_nhwc(conv_a ? &maps.a[sg] : &maps.b[0], dt, plane, dims, strides, lower, upper, (uint32_t)che,
                              (uint32_t)(conv_a ? kBM : bke), trav, &err))
        return fail(RB_UNSUPPORTED, "implicit operand (im2col): " + err);
    }
  }
  for (int s = 0; s < nseg; ++s) {
    if (!conv_a && !encode_operand(&maps.a[s], a_src[seg_a[s]], oa, kBM, &err)) return fail(RB_UNSUPPORTED, "A: " + err);
    if (!conv_b && !encode_operand(&maps.b[s], b_src[seg_b[s]], ob, bn / ctas, &err)) return fail(RB_UNSUPPORTED, "B: " + err);
  }

  GemmParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.G = p->g; kp.M = p->m; kp.N = p->n; kp.K = p->k;
  kp.bn = bn;
  kp.splits = splits;
  kp.tiles_m = (p->m + kBM * ctas - 1) / (kBM * ctas);
  kp.tiles_n = (p->n + bn - 1) / bn;
  kp.kblocks = (p->k + bke - 1) / bke;
  kp.nseg = nseg;
  kp.idesc = make_idesc(cfmt, fmt, fmt_b == 0xffffffffu ? fmt : fmt_b, a_mn ? 1u : 0u, b_mn ? 1u : 0u, (uint32_t)(kBM * ctas), (uint32_t)bn);
  kp.acc_is_int = is_int ? 1 : 0;
  EpiParams ep;
  memset(&ep, 0, sizeof(ep));
  if (epi) {
    ep.flags = epi->flags; ep.alpha = epi->alpha; ep.out_recip = epi->out_recip;
    ep.mid_type = epi->mid_type; ep.bias_type = epi->bias_type;
    ep.col_scale = epi->col_scale; ep.bias = epi->bias;
    ep.clip_lo = epi->clip_lo; ep.clip_hi = epi->clip_hi;
    ep.in_zero = epi->in_zero; ep.out_zero = (epi->flags & RB_EPI_ZP_OUT) ? epi->out_zero : 0;
    ep.residual = epi->residual; ep.res_type = epi->res_type;
    ep.unary = (epi->flags & RB_EPI_UNARY) ? epi->unary : 0;
  }
  if (p->store_method == 1) {
    // the kernel's result is rounded to C's type and added to what C holds, like an atomic add of the stored value
    ep.flags |= RB_EPI_RESIDUAL;
    ep.residual = c; ep.res_type = p->c_type;
    if (!(ep.flags & RB_EPI_ROUND_MID)) { ep.flags |= RB_EPI_ROUND_MID; ep.mid_type = p->c_type; }
  }
  const size_t es_c = dtype_bytes(p->c_type);
  void* partial = splits > 1 ? static_cast<void*>(wsb + ws.partial_off) : nullptr;
  if (splits > 1 && conva && conva->c_rows_per_img > 0)
    return fail(RB_UNSUPPORTED, "a channel-major result cannot be combined with a K split");
  if (splits > 1) {
    // every K range writes raw accumulators into its own plane; the reduction applies the epilogue
    kp.c = partial;
    kp.c_type = is_int ? RB_I32 : RB_F32;
    kp.c_stride_m = p->n; kp.c_stride_n = 1;
    kp.c_stride_g = (long long)p->m * p->n;
    kp.split_stride = (long long)p->g * p->m * p->n;
    kp.vec_ok = (p->n % 4 == 0) ? 1 : 0;
    kp.c_tma = (kp.vec_ok && !cfg.plain_stores) ? 1 : 0;   // planes are stored like a C of splits * g groups
  } else {
    kp.c = c;
    kp.c_type = p->c_type;
    if (p->trans_c) { kp.c_stride_m = 1; kp.c_stride_n = p->m; } else { kp.c_stride_m = p->n; kp.c_stride_n = 1; }
    kp.c_stride_g = (long long)p->m * p->n;
    if (chain)   // signed distance from group 0's result to group 1's, in elements
      kp.c_stride_g = (reinterpret_cast<intptr_t>(chain->c2) - reinterpret_cast<intptr_t>(c)) / (intptr_t)es_c;
    kp.vec_ok = (!p->trans_c && ((size_t)p->n * es_c) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0) ? 1 : 0;
    kp.c_tma = (kp.vec_ok && !cfg.plain_stores) ? 1 : 0;
    if (conva && conva->c_rows_per_img > 0) {   // NKHW result: strided element stores, coalesced along the pixels
      kp.c_rows_per_img = conva->c_rows_per_img;
      kp.c_img_stride = conva->c_img_stride;
      kp.c_stride_m = 1;
      kp.c_stride_n = conva->c_col_stride;
      kp.vec_ok = 0;
      kp.c_tma = 0;
    }
    kp.epi = ep;
  }
  if (kp.c_tma) {
    const int st_type = kp.c_type;                      // what the kernel stores: C's type, or raw planes
    const size_t es_st = dtype_bytes(st_type);
    const CUtensorMapDataType cdt = st_type == RB_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                    : st_type == RB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                    : st_type == RB_F32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                    : st_type == RB_I32  ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                                         : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const uint64_t cdims[3] = {(uint64_t)p->n, (uint64_t)p->m, (uint64_t)p->g * splits};
    const uint64_t cstrides[2] = {(uint64_t)p->n * es_st, chain ? chain_stride[2] : (uint64_t)p->m * p->n * es_st};
    const uint32_t cbox[3] = {(uint32_t)(kRowBytes / es_st), 32u, 1u};
    void* cbase = (chain && (chain_flip & 4)) ? chain->c2 : kp.c;
    if (!encode_tiled(&maps.c, cdt, 3, cbase, cdims, cstrides, cbox, CU_TENSOR_MAP_SWIZZLE_128B, &err))
      return fail(RB_UNSUPPORTED, "C: " + err);
  }
  kp.status = dev->status_word;
  kp.stages = stages;
  kp.kpr = cfg.kpr;
  kp.probe = kProbeBuild ? (t_variant >> 24) & 7 : 0;
  kp.wait_cycles = t_wait_cycles;
  if (t_stall_launches > 0) { kp.stall = 1; --t_stall_launches; }
  if (conva) {
    kp.conva.enabled = conv_a ? 1 : 2; kp.conva.P = conva->P; kp.conva.Q = conva->Q; kp.conva.X = conva->X;
    kp.conva.cchunks = conva->C / bke;
    kp.conva.stride_h = conva->stride_h; kp.conva.stride_w = conva->stride_w;
    kp.conva.dil_h = conva->dil_h; kp.conva.dil_w = conva->dil_w; kp.conva.pad_h = conva->pad_h; kp.conva.pad_w = conva->pad_w;
  }
  kp.a_fused = a_fused ? 1 : 0;
  kp.b_fused = b_fused ? 1 : 0;

  if (chain) {
    if ((size_t)kp.tiles_m * kp.tiles_n * ctas * 4 * sizeof(unsigned int) > chain->flags_bytes)
      return fail(RB_UNSUPPORTED, "chained launch: too many tiles for the flag words");
    static std::atomic<unsigned int> next_chain_token{0xc4a10001u};
    kp.chain_flags = chain->flags;
    kp.chain_token = next_chain_token.fetch_add(1, std::memory_order_relaxed);
    kp.chain_flip = chain_flip;
  }
  const long long num_tiles = (long long)kp.G * kp.tiles_m * kp.tiles_n;
  const long long num_items = num_tiles * splits;
  if (num_items > 0x7fffffffLL) return fail(RB_UNSUPPORTED, "too many tiles");
  // the stream-K split was planned for a B200's SM count; on anything else every tile is computed whole
  const bool use_sk = cfg.sk_tiles > 0 && dev->sm_count == planned_sms();
  kp.dp_tiles = use_sk ? cfg.dp_tiles : (int)num_tiles;
  kp.sk_tiles = use_sk ? cfg.sk_tiles : 0;
  if (use_sk) {
    kp.sk_partial = wsb + ws.sk_off;
    kp.sk_flags = reinterpret_cast<unsigned int*>(wsb + ws.sk_flags_off);
    static std::atomic<unsigned int> next_token{0x5eed0001u};
    kp.sk_token = next_token.fetch_add(1, std::memory_order_relaxed);
  }

  // the instantiation with the fused elementwise code only when this launch has such work (see gemm_tcgen05_kernel)
  const bool epi_kernel = kp.epi.flags != 0;
  GemmKernel kern = epi_kernel ? (ctas == 2 ? pick_kernel<2, true>(kind, a_mn, b_mn) : pick_kernel<1, true>(kind, a_mn, b_mn))
                               : (ctas == 2 ? pick_kernel<2, false>(kind, a_mn, b_mn) : pick_kernel<1, false>(kind, a_mn, b_mn));
  const bool kernel_epi_vec = splits == 1 && epi_vec;  // with a K split the reduction kernel applies the epilogue
  const int smem = ctas == 2 ? GemmSmemLayout<2>::total(stages, bn, kernel_epi_vec) : GemmSmemLayout<1>::total(stages, bn, kernel_epi_vec);
  {
    const RbStatus sst = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem);
    if (sst != RB_SUCCESS) return sst;
  }

  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.blockDim = dim3(kGemmThreads, 1, 1);
  lc.dynamicSmemBytes = (size_t)smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  lc.attrs = attr;
  if (ctas == 2) {
    attr[lc.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[lc.numAttrs].val.clusterDim.x = 2; attr[lc.numAttrs].val.clusterDim.y = 1; attr[lc.numAttrs].val.clusterDim.z = 1;
    ++lc.numAttrs;
    const int pairs = dev->sm_count / 2;
    lc.gridDim = dim3((unsigned)(2 * (int)std::min<long long>(num_items, pairs)), 1, 1);
  } else {
    lc.gridDim = dim3((unsigned)std::min<long long>(num_items, dev->sm_count), 1, 1);
  }
  if (capture) {
    static_assert(sizeof(GemmTensorMaps) + sizeof(GemmParams) + 64 <= sizeof(capture->params), "parameter block too small");
    memset(capture, 0, sizeof(*capture));
    const std::string sym = kernel_symbol(kind, kind == kKindTF32 ? false : a_mn, kind == kKindTF32 ? false : b_mn, ctas, epi_kernel);
    snprintf(capture->symbol, sizeof(capture->symbol), "%s", sym.c_str());
    capture->grid = lc.gridDim.x;
    capture->block = kGemmThreads;
    capture->cluster = (uint32_t)ctas;
    capture->dynamic_smem = (uint32_t)smem;
    capture->param_count = 2;
    capture->param_offset[0] = 0;
    capture->param_size[0] = (uint32_t)sizeof(GemmTensorMaps);
    capture->param_offset[1] = (uint32_t)((sizeof(GemmTensorMaps) + 63) / 64 * 64);
    capture->param_size[1] = (uint32_t)sizeof(GemmParams);
    kp.trace = nullptr;
    memcpy(capture->params + capture->param_offset[0], &maps, sizeof(maps));
    memcpy(capture->params + capture->param_offset[1], &kp, sizeof(kp));
    return RB_SUCCESS;
  }
  kp.trace = trace_buffer((size_t)lc.gridDim.x * 16);
  RB_CUDA_TRY(cudaLaunchKernelEx(&lc, kern, maps, kp));
  count_launch();
  if (splits > 1) {
    const long long total = (long long)p->g * p->m * p->n;
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)dev->sm_count * 8);
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(partial, splits, total, p->g, p->m, p->n, c, p->c_type,
                                                     p->trans_c ? 1 : 0, is_int ? 1 : 0, ep);
    count_launch();
  }
  return RB_SUCCESS;
}

// ---- the kernels as a loadable binary --------------------------------------------------------------------------------
// The image is the cubin that nvcc makes of csrc/cubin/gemm_kernels.cu (every instantiation of gemm_tcgen05_kernel
// for sm_100a), linked into the library as data.
extern "C" const unsigned char rb_gemm_cubin_start[];
extern "C" const unsigned char rb_gemm_cubin_end[];

extern "C" RbStatus rbGetKernelBinary(const void** image, size_t* size) {
  if (!image && !size) return rb::fail(RB_INVALID_PARAM, "image and size are both NULL");
  if (image) *image = rb_gemm_cubin_start;
  if (size) *size = (size_t)(rb_gemm_cubin_end - rb_gemm_cubin_start);
  return RB_SUCCESS;
}

extern "C" RbStatus rbGemmEncodeLaunch(const RbGemmProblem* p, const RbEpilogue* epi, const void* a, const void* b, void* c,
                                       RbKernelLaunch* out) {
  if (!out) return rb::fail(RB_INVALID_PARAM, "out is NULL");
  return rb::gemm_run(p, epi, a, b, c, nullptr, 0, nullptr, nullptr, out);
}

// ---- rbGemmNoAlloc ------------------------------------------------------------------------------------
// Scratch for callers that may not allocate device memory: one fixed array inside the library image. Every GPU
// that loads the library carries it until the process exits; all calls share it.
namespace {
constexpr size_t kNoAllocScratchBytes = RB_NO_ALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 16;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kNoAllocMaxDevices];   // nullptr until a lookup on that device has succeeded
}  // namespace

extern "C" RbStatus rbGemmNoAlloc(const RbGemmProblem* p, const RbEpilogue* epi, const void* a, const void* b, void* c,
                                  void* stream) {
  RbStatus st = rb::check_problem(p);
  if (st != RB_SUCCESS) return st;
  const size_t need = rbGemmWorkspaceSize(p);
  if (need > kNoAllocScratchBytes)
    return rb::fail(RB_WORKSPACE_TOO_SMALL,
                    "rbGemmNoAlloc: this problem needs " + std::to_string(need) + " bytes of scratch, the built-in "
                    "scratch holds " + std::to_string(kNoAllocScratchBytes) + "; use rbGemm with a caller workspace");
  int dev = 0;
  RB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return rb::fail(RB_CUDA_ERROR, "device index out of range");
  // In host code the array's name is only a handle for the runtime, not a device address: the address the kernels
  // get is looked up per device, with that device current. Only a successful lookup is remembered; a failed one
  // (for instance a first call made while a stream capture was open) is reported and tried again by the next call.
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void* ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr)
        return rb::fail(RB_CUDA_ERROR, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
  }
  return rbGemm(p, epi, a, b, c, need ? scratch : nullptr, need ? kNoAllocScratchBytes : 0, stream);
}

// ---- rbGemmGemm -------------------------------------------------------------------------------------------
// O = (A . B1) . B2 with the intermediate rounded to the element type: what rocMLIR's attention skeleton computes
// with the softmax removed (mlir/lib/Dialect/Rock/Transforms/GridwiseGemmToBlockwise.cpp:1790-1813, 2162-2165).
// With k1 and n2 at most 128 (the shapes of that skeleton) it runs on the attention kernel in one launch: S = A . B1
// in tensor memory, rounded to the element type in place, second product straight from there; no workspace. Larger
// inner extents do not fit the SM (O alone would be 128 x n2 f32 in TMEM): the intermediate (M x N1, element type)
// goes through the caller's workspace, small enough to stay in L2 - as one chained launch of the GEMM kernel when
// k1 = n1 = n2 (see below), else as two launches. Variant bit 27 forces the two-launch form.
// Flag words of the chained form: four per (128-row block, tile of columns), for tiles of 32 columns or more.
static size_t chain_flag_bytes(int m, int n1) {
  return rb::align_up((size_t)((m + 127) / 128) * ((n1 + 31) / 32) * 4 * sizeof(unsigned int), 256);
}

extern "C" size_t rbGemmGemmWorkspaceSize(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type) {
  if (g <= 0 || m <= 0 || k1 <= 0 || n1 <= 0 || n2 <= 0 || !rb::dtype_bytes(data_type)) return 0;
  // (the one-launch form needs none of it; the size is reported for the two-launch form so that a caller who sized
  // its buffer once can switch forms with the variant word)
  RbGemmProblem p1 = {g, m, n1, k1, 0, 0, 0, data_type, data_type, 0};
  RbGemmProblem p2 = {g, m, n2, n1, 0, 0, 0, data_type, data_type, 0};
  const size_t mid = rb::align_up((size_t)g * m * n1 * rb::dtype_bytes(data_type), 256);
  return mid + std::max(rbGemmWorkspaceSize(&p1), rbGemmWorkspaceSize(&p2)) + chain_flag_bytes(m, n1);
}

extern "C" RbStatus rbGemmGemm(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type,
                               const void* a, const void* b1, const void* b2, void* o, void* workspace,
                               size_t workspace_bytes, void* stream) {
  if (!(data_type == RB_F16 || data_type == RB_BF16 || data_type == RB_F32))
    return rb::fail(RB_UNSUPPORTED, "gemm+gemm exists for f16, bf16 and f32");
  const size_t need = rbGemmGemmWorkspaceSize(g, m, k1, n1, n2, data_type);
  if (need == 0) return rb::fail(RB_INVALID_PARAM, "sizes must be positive");
  if (rb::gemm_gemm_on_chip_applicable(k1, n1, n2, data_type) && !((rbGetGemmVariant() >> 27) & 1))
    return rb::gemm_gemm_on_chip(g, m, k1, n1, n2, data_type, a, b1, b2, o, stream);
  if (!workspace || workspace_bytes < need)
    return rb::fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(need) + " bytes required");
  RbGemmProblem p1 = {g, m, n1, k1, 0, 0, 0, data_type, data_type, 0};
  RbGemmProblem p2 = {g, m, n2, n1, 0, 0, 0, data_type, data_type, 0};
  const size_t mid = rb::align_up((size_t)g * m * n1 * rb::dtype_bytes(data_type), 256);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  // Equal inner extents (k1 = n1 = n2), one group, 16-bit: ONE launch of the GEMM kernel over a two-group problem whose
  // second group reads the first group's result; the tiles of the second product start as soon as the row block of the
  // intermediate they read is complete, so there is no drain and refill between the products. Variant bit 27 keeps
  // the two-launch form; shapes or pointers the chained form does not take fall through to it.
  if (g == 1 && k1 == n1 && n1 == n2 && data_type != RB_F32 && !((rbGetGemmVariant() >> 27) & 1)) {
    const size_t fb = chain_flag_bytes(m, n1);
    RbGemmProblem pc = {2, m, n1, k1, 0, 0, 0, data_type, data_type, 0};
    rb::GemmChain ch = {b2, o, reinterpret_cast<unsigned int*>(ws + need - fb), fb};
    rb::t_chain = &ch;
    const RbStatus cst = rbGemm(&pc, nullptr, a, b1, ws, nullptr, 0, stream);
    rb::t_chain = nullptr;
    if (cst != RB_UNSUPPORTED) return cst;
  }
  RbStatus st = rbGemm(&p1, nullptr, a, b1, ws, ws + mid, workspace_bytes - mid, stream);
  if (st != RB_SUCCESS) return st;
  return rbGemm(&p2, nullptr, ws, b2, o, ws + mid, workspace_bytes - mid, stream);
}
