// Convolutions with three image dimensions (rocmlir-gen builds them for layouts with three image letters,
// mlir/tools/rocmlir-gen/rocmlir-gen.cpp:3545-3581; ConvGenerator keeps a DEPTH entry in every per-dimension
// vector, mlir/lib/Dialect/Rock/Generator/ConvGenerator.cpp:592-607).
//
// The reference lowers them through the same coordinate maps as the 2-D case with one more merged dimension. Here
// the depth is folded into a 2-D problem so that the tcgen05 paths of rbConv do all the arithmetic:
//
//   in2[g, (n,do), h, w, (z,c)] = in[n, g, c, do*stride_d + z*dil_d - pad_d, h, w]     (zero outside the image)
//   fil2[g, k, y, x, (z,c)]     = fil[g, k, c, z, y, x]
//   out2[g, (n,do), ho, wo, k]  = out[n, g, k, do, ho, wo]
//
// and out2 = conv2d(in2, fil2) with N*Do images and Z*C channels. Forward and backward weight gather in2 with one
// pass; backward data runs the 2-D backward-data kernels into in2 and then sums, for every input voxel, the taps z
// whose (d + pad_d - z*dil_d) is a multiple of stride_d with the quotient inside the output depth (the 2-D kernels
// leave in2 in f32 for that, so the sum rounds once). A problem with all depths equal to 1 is the 2-D problem on
// the same bytes and is passed through.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string.h>

#include <string>

#include "lib_state.h"

namespace rb {
namespace {

// Dense row-major tensor of `size` on one side, strided tensor on the other. With jd >= 0 the strided offset also
// gets d * s_d with d = coord[jd] * sd + coord[jz] * dd - pd, and the element is zero (gather) when d is outside.
struct Remap7 {
  long long size[7];
  long long stride[7];
  int jd, jz;
  long long sd, dd, pd, D, s_d;
};

template <int ES>
__global__ void remap7_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, Remap7 r, int to_dense) {
  long long total = 1;
#pragma unroll
  for (int k = 0; k < 7; ++k) total *= r.size[k];
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, off = 0, cd = 0, cz = 0;
#pragma unroll
    for (int k = 6; k >= 0; --k) {
      const long long q = rem / r.size[k];
      const long long c = rem - q * r.size[k];
      off += c * r.stride[k];
      if (k == r.jd) cd = c;
      if (k == r.jz) cz = c;
      rem = q;
    }
    bool ok = true;
    if (r.jd >= 0) {
      const long long d = cd * r.sd + cz * r.dd - r.pd;
      ok = d >= 0 && d < r.D;
      off += d * r.s_d;
    }
    if (to_dense) {
      if (ES == 1) dst[i] = ok ? src[off] : (uint8_t)0;
      if (ES == 2) reinterpret_cast<uint16_t*>(dst)[i] = ok ? reinterpret_cast<const uint16_t*>(src)[off] : (uint16_t)0;
      if (ES == 4) reinterpret_cast<uint32_t*>(dst)[i] = ok ? reinterpret_cast<const uint32_t*>(src)[off] : 0u;
    } else if (ok) {
      if (ES == 1) dst[off] = src[i];
      if (ES == 2) reinterpret_cast<uint16_t*>(dst)[off] = reinterpret_cast<const uint16_t*>(src)[i];
      if (ES == 4) reinterpret_cast<uint32_t*>(dst)[off] = reinterpret_cast<const uint32_t*>(src)[i];
    }
  }
}

struct FoldParams {
  long long N, D, H, W, G, C;          // the input gradient, iterated in this order
  long long s_n, s_d, s_h, s_w, s_g, s_c;   // its strides in the caller's layout
  long long Do, Z, sd, dd, pd;
};

__device__ __forceinline__ void st_f32(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_f32(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void st_f32(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

// din[n,g,c,d,h,w] = sum_z din2[g,(n,do),h,w,(z,c)] over the taps with do = (d + pd - z*dd) / sd exact and in range;
// din2 is the f32 gradient of the folded 2-D problem, so the sum rounds once into the element type
template <typename T>
__global__ void depth_fold_kernel(const float* __restrict__ din2, T* __restrict__ din, FoldParams f) {
  const long long total = f.N * f.D * f.H * f.W * f.G * f.C;
  const long long zc = f.Z * f.C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long rem = i;
    const long long c = rem % f.C; rem /= f.C;
    const long long g = rem % f.G; rem /= f.G;
    const long long w = rem % f.W; rem /= f.W;
    const long long h = rem % f.H; rem /= f.H;
    const long long d = rem % f.D;
    const long long n = rem / f.D;
    float acc = 0.0f;
    for (long long z = 0; z < f.Z; ++z) {
      const long long t = d + f.pd - z * f.dd;
      if (t < 0 || t % f.sd) continue;
      const long long dout = t / f.sd;
      if (dout >= f.Do) continue;
      acc += din2[((((g * f.N + n) * f.Do + dout) * f.H + h) * f.W + w) * zc + z * f.C + c];
    }
    st_f32(din, n * f.s_n + d * f.s_d + h * f.s_h + w * f.s_w + g * f.s_g + c * f.s_c, acc);
  }
}

size_t up256(size_t x) { return (x + 255) / 256 * 256; }

// Strides of the named dimensions of a tensor stored in `layout` order; digits 0 1 2 alias the image letters.
bool strides6(const char* layout, const char* letters, const long long* sizes, long long* strides) {
  if (!layout || strlen(layout) != 6) return false;
  long long acc = 1;
  bool seen[6] = {false, false, false, false, false, false};
  for (int pos = 5; pos >= 0; --pos) {
    char ch = layout[pos];
    if (ch >= '0' && ch <= '2') ch = letters[6 + (ch - '0')];
    const char* f = static_cast<const char*>(memchr(letters, ch, 6));
    if (!f) return false;
    const int idx = (int)(f - letters);
    if (seen[idx]) return false;
    seen[idx] = true;
    strides[idx] = acc;
    acc *= sizes[idx];
  }
  return true;
}

long long out_extent(long long in, long long fil, long long pl, long long pr, long long stride, long long dil) {
  return (in + pl + pr - (fil - 1) * dil - 1) / stride + 1;
}

struct Plan3d {
  bool flat;                 // all depths 1: the 2-D problem on the same bytes
  bool widen;                // the 2-D backward-data result is asked for in f32
  RbConvProblem q;           // the 2-D problem that does the arithmetic
  long long fs[6], is[6], os[6];   // strides for (g,k,c,z,y,x), (n,g,c,d,h,w), (n,g,k,d,h,w)
  size_t in2_bytes, fil2_bytes, out2_bytes, conv_ws;
  size_t in2_off, fil2_off, out2_off, conv_off, total;
};

// Removes the depth letter (or its digit alias) from a 6-letter layout.
bool drop_letter(const char* layout, char letter, char digit, char* out5) {
  int n = 0;
  for (int i = 0; i < 6; ++i) {
    char ch = layout[i];
    if (ch == letter || ch == digit) continue;
    if (n == 5) return false;
    out5[n++] = ch;
  }
  out5[n] = 0;
  return n == 5;
}

RbStatus make_plan3d(const RbConv3dProblem* p, Plan3d* pl) {
  if (!p) return fail(RB_INVALID_PARAM, "problem is NULL");
  if (p->n <= 0 || p->g <= 0 || p->c <= 0 || p->k <= 0 || p->d <= 0 || p->h <= 0 || p->w <= 0 || p->z <= 0 ||
      p->y <= 0 || p->x <= 0 || p->stride_d <= 0 || p->stride_h <= 0 || p->stride_w <= 0 || p->dil_d <= 0 ||
      p->dil_h <= 0 || p->dil_w <= 0 || p->pad_d < 0 || p->pad_h < 0 || p->pad_w < 0 || p->pad_d_r < 0 ||
      p->pad_h_r < 0 || p->pad_w_r < 0)
    return fail(RB_INVALID_PARAM, "convolution sizes must be positive (paddings non-negative)");
  if (p->direction < 0 || p->direction > 2) return fail(RB_INVALID_PARAM, "direction must be 0 (fwd), 1 (bwd data), 2 (bwd weight)");
  const long long dout = out_extent(p->d, p->z, p->pad_d, p->pad_d_r, p->stride_d, p->dil_d);
  const long long ho = out_extent(p->h, p->y, p->pad_h, p->pad_h_r, p->stride_h, p->dil_h);
  const long long wo = out_extent(p->w, p->x, p->pad_w, p->pad_w_r, p->stride_w, p->dil_w);
  if (dout <= 0 || ho <= 0 || wo <= 0) return fail(RB_INVALID_PARAM, "the filter does not fit the padded image");
  if (p->dout != dout || p->ho != ho || p->wo != wo)
    return fail(RB_INVALID_PARAM, "dout/ho/wo must equal (in + padL + padR - (fil-1)*dil - 1)/stride + 1 = " +
                                      std::to_string(dout) + " x " + std::to_string(ho) + " x " + std::to_string(wo));
  const int t = p->data_type;
  const bool f8 = t == RB_F8E4M3 || t == RB_F8E5M2;
  if (!(t == RB_F32 || t == RB_F16 || t == RB_BF16 || t == RB_I8 || f8)) return fail(RB_INVALID_PARAM, "unsupported element type");
  if ((t == RB_I8 || f8) && p->direction != 0)
    return fail(RB_UNSUPPORTED, "8-bit convolutions exist in the forward direction only (RockOps.td:101-134, ConvGenerator.cpp:631-638)");
  const long long fsz[6] = {p->g, p->k, p->c, p->z, p->y, p->x};
  const long long isz[6] = {p->n, p->g, p->c, p->d, p->h, p->w};
  const long long osz[6] = {p->n, p->g, p->k, dout, ho, wo};
  // letters, then the letters the digits 0 1 2 stand for (ConvGenerator.cpp:622-627)
  if (!strides6(p->fil_layout, "gkczyxyxz", fsz, pl->fs)) return fail(RB_INVALID_PARAM, "fil_layout must be a permutation of gkczyx");
  if (!strides6(p->in_layout, "ngcdhwhwd", isz, pl->is)) return fail(RB_INVALID_PARAM, "in_layout must be a permutation of ngcdhw");
  if (!strides6(p->out_layout, "ngkdhwhwd", osz, pl->os)) return fail(RB_INVALID_PARAM, "out_layout must be a permutation of ngkdhw");

  RbConvProblem& q = pl->q;
  memset(&q, 0, sizeof(q));
  q.g = p->g; q.k = p->k; q.h = p->h; q.w = p->w; q.y = p->y; q.x = p->x;
  q.stride_h = p->stride_h; q.stride_w = p->stride_w; q.dil_h = p->dil_h; q.dil_w = p->dil_w;
  q.pad_h = p->pad_h; q.pad_w = p->pad_w; q.pad_h_r = p->pad_h_r; q.pad_w_r = p->pad_w_r;
  q.ho = (int)ho; q.wo = (int)wo;
  q.data_type = t; q.direction = p->direction; q.f32_mode = p->f32_mode;
  pl->flat = p->d == 1 && p->z == 1 && p->pad_d == 0 && p->pad_d_r == 0;
  pl->in2_bytes = pl->fil2_bytes = pl->out2_bytes = 0;
  if (pl->flat) {
    q.n = p->n; q.c = p->c;
    if (!drop_letter(p->fil_layout, 'z', '2', q.fil_layout) || !drop_letter(p->in_layout, 'd', '2', q.in_layout) ||
        !drop_letter(p->out_layout, 'd', '2', q.out_layout))
      return fail(RB_INVALID_PARAM, "layouts must name the depth dimension once");
    // the 2-D entry point spells the image letters, not their digit aliases
    for (char* s : {q.fil_layout, q.in_layout, q.out_layout})
      for (int i = 0; i < 5; ++i) {
        const bool fil = s == q.fil_layout;
        if (s[i] == '0') s[i] = fil ? 'y' : 'h';
        if (s[i] == '1') s[i] = fil ? 'x' : 'w';
      }
  } else {
    const long long n2 = (long long)p->n * dout, c2 = (long long)p->z * p->c;
    if (n2 > 0x7fffffffLL || c2 > 0x7fffffffLL) return fail(RB_UNSUPPORTED, "folded extent exceeds 2^31");
    q.n = (int)n2; q.c = (int)c2;
    strcpy(q.fil_layout, "gkyxc");
    strcpy(q.in_layout, "gnhwc");     // group outermost: each group's activations are a [pixels][channels] matrix
    strcpy(q.out_layout, "gnhwk");
    const size_t es = dtype_bytes(t), es_o = dtype_bytes(t == RB_I8 ? RB_I32 : f8 ? RB_F32 : t);
    pl->in2_bytes = (size_t)n2 * p->h * p->w * p->g * c2 * (p->direction == 1 ? 4 : es);
    pl->fil2_bytes = (size_t)p->g * p->k * p->y * p->x * c2 * es;
    pl->out2_bytes = (size_t)n2 * ho * wo * p->g * p->k * es_o;
  }
  pl->widen = !pl->flat && p->direction == 1 && t != RB_F32;   // backward data: f32 gradient of the folded problem
  pl->conv_ws = conv_workspace_bytes(&q, pl->widen ? RB_F32 : -1);
  size_t off = 0;
  pl->in2_off = off; off += up256(pl->in2_bytes);
  pl->fil2_off = off; off += up256(pl->fil2_bytes);
  pl->out2_off = off; off += up256(pl->out2_bytes);
  pl->conv_off = off; off += up256(pl->conv_ws);
  pl->total = off;
  return RB_SUCCESS;
}

template <typename K, typename... Args>
void launch3(size_t es, int blocks, cudaStream_t st, K k1, K k2, K k4, Args... args) {
  if (es == 1) k1<<<blocks, 256, 0, st>>>(args...);
  else if (es == 2) k2<<<blocks, 256, 0, st>>>(args...);
  else k4<<<blocks, 256, 0, st>>>(args...);
}

}  // namespace
}  // namespace rb

using namespace rb;

extern "C" size_t rbConv3dWorkspaceSize(const RbConv3dProblem* p) {
  Plan3d pl;
  if (make_plan3d(p, &pl) != RB_SUCCESS) return 0;
  return pl.total;
}

extern "C" RbStatus rbConv3d(const RbConv3dProblem* p, void* filter, void* input, void* output, void* workspace,
                             size_t workspace_bytes, void* stream_v) {
  Plan3d pl;
  RbStatus st = make_plan3d(p, &pl);
  if (st != RB_SUCCESS) return st;
  if (!filter || !input || !output) return fail(RB_INVALID_PARAM, "filter, input and output must be device pointers");
  if (pl.total > 0 && (!workspace || workspace_bytes < pl.total))
    return fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(pl.total) + " bytes required");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (pl.flat) return rbConv(&pl.q, filter, input, output, ws + pl.conv_off, pl.conv_ws, stream_v);
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int blocks = dev->sm_count * 8;
  const int t = p->data_type;
  const size_t es = dtype_bytes(t), es_o = dtype_bytes(t == RB_I8 ? RB_I32 : (t == RB_F8E4M3 || t == RB_F8E5M2) ? RB_F32 : t);
  uint8_t* in2 = ws + pl.in2_off;
  uint8_t* fil2 = ws + pl.fil2_off;
  uint8_t* out2 = ws + pl.out2_off;

  auto remap = [&](const void* src, void* dst, const Remap7& r, bool to_dense, size_t esz) {
    launch3(esz, blocks, stream, remap7_kernel<1>, remap7_kernel<2>, remap7_kernel<4>, static_cast<const uint8_t*>(src),
            static_cast<uint8_t*>(dst), r, to_dense ? 1 : 0);
    count_launch();
  };
  // in2 [g][(n,do)][h][w][(z,c)]
  Remap7 r_in;
  {
    const long long size[7] = {p->g, p->n, p->dout, p->h, p->w, p->z, p->c};
    const long long stride[7] = {pl.is[1], pl.is[0], 0, pl.is[4], pl.is[5], 0, pl.is[2]};
    memcpy(r_in.size, size, sizeof(size));
    memcpy(r_in.stride, stride, sizeof(stride));
    r_in.jd = 2; r_in.jz = 5;
    r_in.sd = p->stride_d; r_in.dd = p->dil_d; r_in.pd = p->pad_d; r_in.D = p->d; r_in.s_d = pl.is[3];
  }
  // fil2 [g][k][y][x][(z,c)]
  Remap7 r_fil;
  {
    const long long size[7] = {p->g, p->k, p->y, p->x, p->z, p->c, 1};
    const long long stride[7] = {pl.fs[0], pl.fs[1], pl.fs[4], pl.fs[5], pl.fs[3], pl.fs[2], 0};
    memcpy(r_fil.size, size, sizeof(size));
    memcpy(r_fil.stride, stride, sizeof(stride));
    r_fil.jd = -1; r_fil.jz = -1; r_fil.sd = r_fil.dd = 1; r_fil.pd = 0; r_fil.D = 1; r_fil.s_d = 0;
  }
  // out2 [g][(n,do)][ho][wo][k]
  Remap7 r_out = r_fil;
  {
    const long long size[7] = {p->g, p->n, p->dout, p->ho, p->wo, p->k, 1};
    const long long stride[7] = {pl.os[1], pl.os[0], pl.os[3], pl.os[4], pl.os[5], pl.os[2], 0};
    memcpy(r_out.size, size, sizeof(size));
    memcpy(r_out.stride, stride, sizeof(stride));
  }
  uint8_t* cws = ws + pl.conv_off;
  if (p->direction == 0) {
    remap(input, in2, r_in, true, es);
    remap(filter, fil2, r_fil, true, es);
    st = rbConv(&pl.q, fil2, in2, out2, cws, pl.conv_ws, stream_v);
    if (st != RB_SUCCESS) return st;
    remap(out2, output, r_out, false, es_o);
  } else if (p->direction == 2) {
    remap(input, in2, r_in, true, es);
    remap(output, out2, r_out, true, es);
    st = rbConv(&pl.q, fil2, in2, out2, cws, pl.conv_ws, stream_v);
    if (st != RB_SUCCESS) return st;
    remap(fil2, filter, r_fil, false, es);
  } else {
    remap(filter, fil2, r_fil, true, es);
    remap(output, out2, r_out, true, es);
    st = conv_run(&pl.q, pl.widen ? RB_F32 : -1, fil2, in2, out2, cws, pl.conv_ws, stream_v);
    if (st != RB_SUCCESS) return st;
    FoldParams f;
    f.N = p->n; f.D = p->d; f.H = p->h; f.W = p->w; f.G = p->g; f.C = p->c;
    f.s_n = pl.is[0]; f.s_g = pl.is[1]; f.s_c = pl.is[2]; f.s_d = pl.is[3]; f.s_h = pl.is[4]; f.s_w = pl.is[5];
    f.Do = p->dout; f.Z = p->z; f.sd = p->stride_d; f.dd = p->dil_d; f.pd = p->pad_d;
    if (t == RB_F32)
      depth_fold_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(in2), static_cast<float*>(input), f);
    else if (t == RB_F16)
      depth_fold_kernel<__half><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(in2), static_cast<__half*>(input), f);
    else
      depth_fold_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(in2),
                                                                   static_cast<__nv_bfloat16*>(input), f);
    count_launch();
  }
  RB_CUDA_TRY(cudaGetLastError());
  return RB_SUCCESS;
}
