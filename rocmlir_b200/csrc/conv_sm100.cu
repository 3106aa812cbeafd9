// rock.conv / rock.conv_bwd_data / rock.conv_bwd_weight as GEMMs on the tcgen05 kernel.
//
// rocMLIR views the three tensors of a convolution as matrices through coordinate maps and runs its GEMM
// kernel on the views (mlir/lib/Dialect/Rock/Transforms/ConvToGemm.cpp:1133-1400 forward / backward weight,
// :770-1131 backward data; sizes in mlir/lib/Dialect/Rock/IR/RockDialect.cpp:509-533). This file does the same
// with explicit matrices: an operand that already is a row-major matrix in its storage layout (NHWC activations
// of a 1x1 stride-1 convolution, a KYXC filter, an NHWK output) is handed to the GEMM as it lies; anything else
// is gathered into (or scattered from) a matrix in the caller's workspace by the kernels below.
//
//   forward      out[(n,ho,wo), k]   = sum_{y,x,c} im2col(in)[(n,ho,wo), (y,x,c)] * fil[k, (y,x,c)]
//   backward wt  fil[k, (y,x,c)]     = sum_{n,ho,wo} out[(n,ho,wo), k] * im2col(in)[(n,ho,wo), (y,x,c)]
//   backward dat in[(n,h,w), c]      = sum_{y,x,k} col2im(out)[(n,h,w), (y,x,k)] * fil[(y,x,k), c]
// Groups are the GEMM batch dimension. Index relation and output-size rule are the reference's
// (in_h = ho*stride + y*dil - pad; mlir/include/mlir/Dialect/Rock/Generator/ConvGenerator.h:98-104).
//
// Implicit GEMM (no im2col matrix in memory) for dense NHWC tensors of one group whose channel count is a multiple
// of 128 bytes: the GEMM producer fetches the im2col tiles itself with TMA im2col descriptors -
//   forward       A from the input (16-bit and 8-bit types; f32 through TF32 planes of the input, hi and lo, which
//                 one pass builds and, for an NCHW input, transposes)
//   backward data A from the output gradient with padding (fil-1)*dil - pad and the filter taps mirrored. With a
//                 stride the problem is cut into one unit-stride problem per class of input pixels (see ClassTable);
//                 only a stride together with a dilation still zero-upsamples the gradient into the workspace
//   backward wt   B from the input (K index = output pixel), A = the NHWK output gradient in place.
#include <cuda_runtime.h>
#include <string.h>

#include <algorithm>
#include <string>

#include "lib_state.h"

namespace rb {
namespace {

struct Dims5 {
  long long size[5];
  long long stride[5];
};

// Copies a 5-D tensor between a strided layout and the dense row-major layout of `size`.
// to_dense: dst[dense] = src[strided]; else dst[strided] = src[dense]. ES = element bytes.
template <int ES>
__global__ void permute5_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, Dims5 d, int to_dense) {
  const long long total = d.size[0] * d.size[1] * d.size[2] * d.size[3] * d.size[4];
  if (total <= 0xffffffffLL) {
    // the usual case: 32-bit index arithmetic (64-bit divisions cost an order of magnitude more)
    const unsigned n = (unsigned)total;
    const unsigned s0 = (unsigned)d.size[0], s1 = (unsigned)d.size[1], s2 = (unsigned)d.size[2], s3 = (unsigned)d.size[3],
                   s4 = (unsigned)d.size[4];
    (void)s0;
    for (unsigned long long i64 = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i64 < n;
         i64 += (unsigned long long)gridDim.x * blockDim.x) {
      const unsigned i = (unsigned)i64;
      unsigned r = i;
      const unsigned i4 = r % s4; r /= s4;
      const unsigned i3 = r % s3; r /= s3;
      const unsigned i2 = r % s2; r /= s2;
      const unsigned i1 = r % s1; r /= s1;
      const long long off = (long long)r * d.stride[0] + (long long)i1 * d.stride[1] + (long long)i2 * d.stride[2] +
                            (long long)i3 * d.stride[3] + (long long)i4 * d.stride[4];
      const long long s = to_dense ? off : (long long)i, t = to_dense ? (long long)i : off;
      if (ES == 1) dst[t] = src[s];
      if (ES == 2) reinterpret_cast<uint16_t*>(dst)[t] = reinterpret_cast<const uint16_t*>(src)[s];
      if (ES == 4) reinterpret_cast<uint32_t*>(dst)[t] = reinterpret_cast<const uint32_t*>(src)[s];
    }
    return;
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i, off = 0;
#pragma unroll
    for (int k = 4; k >= 0; --k) {
      const long long q = r / d.size[k];
      off += (r - q * d.size[k]) * d.stride[k];
      r = q;
    }
    const long long s = to_dense ? off : i, t = to_dense ? i : off;
    if (ES == 1) dst[t] = src[s];
    if (ES == 2) reinterpret_cast<uint16_t*>(dst)[t] = reinterpret_cast<const uint16_t*>(src)[s];
    if (ES == 4) reinterpret_cast<uint32_t*>(dst)[t] = reinterpret_cast<const uint32_t*>(src)[s];
  }
}

// The common permutation - a [pixels][channels] matrix against an NCHW-like tensor - is a batched 2-D transpose:
// dense side [b0][b1][R][C] (C contiguous), strided side with the R run contiguous (stride 1) and the channel at
// stride s_c. 32 x 32 tiles through shared memory keep both sides coalesced; permute5_kernel, which walks the dense
// index and scatters, reaches about a fifth of this kernel's rate on such tensors.
struct Transpose2 {
  long long B0, B1, R, C;          // dense extents
  long long s_b0, s_b1, s_c;       // strided side: strides of b0, b1 and the column; rows have stride 1
};

template <typename T>
__global__ void transpose_tiles_kernel(const T* __restrict__ src, T* __restrict__ dst, Transpose2 t, int to_dense) {
  __shared__ T tile[32][33];
  const long long tiles_r = (t.R + 31) / 32, tiles_c = (t.C + 31) / 32;
  const long long total = t.B0 * t.B1 * tiles_r * tiles_c;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads
  for (long long w = blockIdx.x; w < total; w += gridDim.x) {
    long long rem = w;
    const long long tc = rem % tiles_c; rem /= tiles_c;
    const long long tr = rem % tiles_r; rem /= tiles_r;
    const long long b1 = rem % t.B1, b0 = rem / t.B1;
    const long long r0 = tr * 32, c0 = tc * 32;
    const long long dense0 = ((b0 * t.B1 + b1) * t.R) * t.C;
    const long long strided0 = b0 * t.s_b0 + b1 * t.s_b1;
    if (to_dense) {
      // read the strided side along r (contiguous), write the dense side along c
#pragma unroll
      for (int j = ty; j < 32; j += 8)
        if (c0 + j < t.C && r0 + tx < t.R) tile[j][tx] = src[strided0 + (c0 + j) * t.s_c + r0 + tx];
      __syncthreads();
#pragma unroll
      for (int j = ty; j < 32; j += 8)
        if (r0 + j < t.R && c0 + tx < t.C) dst[dense0 + (r0 + j) * t.C + c0 + tx] = tile[tx][j];
    } else {
#pragma unroll
      for (int j = ty; j < 32; j += 8)
        if (r0 + j < t.R && c0 + tx < t.C) tile[j][tx] = src[dense0 + (r0 + j) * t.C + c0 + tx];
      __syncthreads();
#pragma unroll
      for (int j = ty; j < 32; j += 8)
        if (c0 + j < t.C && r0 + tx < t.R) dst[strided0 + (c0 + j) * t.s_c + r0 + tx] = tile[tx][j];
    }
    __syncthreads();
  }
}

struct GatherParams {
  // matrix: [G][rows = N * P * Q][cols = Y * X * CH], dense, row pitch `pitch` elements
  long long N, G, P, Q, Y, X, CH;
  long long pitch;
  // source tensor (n, g, ch, a, b) strides in elements and image extent
  long long s_n, s_g, s_ch, s_a, s_b;
  long long A, B;
  // index relation
  long long stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
  int transposed;  // 0: a = p*stride + y*dil - pad (im2col); 1: a = (p + pad - y*dil) / stride when divisible (col2im)
};

template <int ES>
__global__ void conv_gather_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, GatherParams g) {
  // Rows, columns and every per-tensor extent fit 32 bits (checked by the plan); only the flat index is 64-bit, so
  // all but the first division are 32-bit.
  const unsigned cols = (unsigned)(g.Y * g.X * g.CH), pitch = (unsigned)g.pitch;
  const unsigned rows = (unsigned)(g.N * g.P * g.Q);
  const unsigned CH = (unsigned)g.CH, X = (unsigned)g.X, Q = (unsigned)g.Q, P = (unsigned)g.P;
  const long long total = g.G * (long long)rows * pitch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned col = (unsigned)(i % pitch);
    const unsigned long long r = (unsigned long long)(i / pitch);
    const unsigned row = (unsigned)(r % rows);
    const unsigned grp = (unsigned)(r / rows);
    bool ok = col < cols;
    long long off = 0;
    if (ok) {
      const unsigned ch = col % CH, t = col / CH;
      const unsigned x = t % X, y = t / X;
      const unsigned q = row % Q, t2 = row / Q;
      const unsigned pp = t2 % P, n = t2 / P;
      int a, b;
      if (!g.transposed) {
        a = (int)(pp * (unsigned)g.stride_h + y * (unsigned)g.dil_h) - (int)g.pad_h;
        b = (int)(q * (unsigned)g.stride_w + x * (unsigned)g.dil_w) - (int)g.pad_w;
      } else {
        const int ta = (int)pp + (int)g.pad_h - (int)(y * (unsigned)g.dil_h), tb = (int)q + (int)g.pad_w - (int)(x * (unsigned)g.dil_w);
        ok = ta >= 0 && tb >= 0 && ta % (int)g.stride_h == 0 && tb % (int)g.stride_w == 0;
        a = ta / (int)g.stride_h;
        b = tb / (int)g.stride_w;
      }
      ok = ok && a >= 0 && a < (int)g.A && b >= 0 && b < (int)g.B;
      off = (long long)n * g.s_n + (long long)grp * g.s_g + (long long)ch * g.s_ch + (long long)a * g.s_a + (long long)b * g.s_b;
    }
    if (ES == 1) dst[i] = ok ? src[off] : (uint8_t)0;
    if (ES == 2) reinterpret_cast<uint16_t*>(dst)[i] = ok ? reinterpret_cast<const uint16_t*>(src)[off] : (uint16_t)0;
    if (ES == 4) reinterpret_cast<uint32_t*>(dst)[i] = ok ? reinterpret_cast<const uint32_t*>(src)[off] : 0u;
  }
}

// The same gather for channel-contiguous sources (NHWC-like: s_ch == 1): one 16-byte vector of channels per thread
// and iteration, index arithmetic once per vector and in 32 bits after the first division. Requires CH * ES and the
// row pitch to be multiples of 16 bytes and 16-byte aligned buffers.
template <int ES>
__global__ void conv_gather_vec_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, GatherParams g) {
  constexpr int VE = 16 / ES;                      // elements per vector
  const unsigned pitch_v = (unsigned)(g.pitch / VE), chv = (unsigned)(g.CH / VE);
  const unsigned rows = (unsigned)(g.N * g.P * g.Q);
  const unsigned X = (unsigned)g.X, Q = (unsigned)g.Q, P = (unsigned)g.P;
  const long long total = g.G * (long long)rows * pitch_v;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned colv = (unsigned)(i % pitch_v);
    const unsigned long long r = (unsigned long long)(i / pitch_v);
    const unsigned row = (unsigned)(r % rows);
    const unsigned grp = (unsigned)(r / rows);
    const unsigned cv = colv % chv, t = colv / chv;
    const unsigned x = t % X, y = t / X;
    const unsigned q = row % Q, t2 = row / Q;
    const unsigned pp = t2 % P, n = t2 / P;
    int a, b;
    bool ok = true;
    if (!g.transposed) {
      a = (int)(pp * (unsigned)g.stride_h + y * (unsigned)g.dil_h) - (int)g.pad_h;
      b = (int)(q * (unsigned)g.stride_w + x * (unsigned)g.dil_w) - (int)g.pad_w;
    } else {
      const int ta = (int)pp + (int)g.pad_h - (int)(y * (unsigned)g.dil_h), tb = (int)q + (int)g.pad_w - (int)(x * (unsigned)g.dil_w);
      ok = ta >= 0 && tb >= 0 && ta % (int)g.stride_h == 0 && tb % (int)g.stride_w == 0;
      a = ta / (int)g.stride_h;
      b = tb / (int)g.stride_w;
    }
    ok = ok && a >= 0 && a < (int)g.A && b >= 0 && b < (int)g.B;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ok) {
      const long long off = (long long)n * g.s_n + (long long)grp * g.s_g + (long long)cv * VE + (long long)a * g.s_a + (long long)b * g.s_b;
      v = __ldg(reinterpret_cast<const uint4*>(src + off * ES));
    }
    reinterpret_cast<uint4*>(dst)[i] = v;
  }
}

// Zero-upsampling of an NHWK tensor for a strided backward-data convolution: out[n][p*sh][q*sw][:] = in[n][p][q][:],
// zeros elsewhere (out is N x ((P-1)*sh+1) x ((Q-1)*sw+1) x CH). One 16-byte vector of channels per thread and step.
__global__ void upsample_nhwc_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int N, int P, int Q, int UP,
                                     int UQ, int chv, int sh, int sw) {
  const long long total = (long long)N * UP * UQ * chv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned cv = (unsigned)(i % chv);
    const unsigned long long r = (unsigned long long)(i / chv);
    const unsigned uq = (unsigned)(r % UQ);
    const unsigned r2 = (unsigned)(r / UQ);
    const unsigned up = r2 % UP, n = r2 / UP;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (up % sh == 0 && uq % sw == 0)
      v = __ldg(in + (((long long)n * P + up / sh) * Q + uq / sw) * chv + cv);
    out[i] = v;
  }
}

// Backward data with a stride, by classes of input pixels. An input pixel h only receives taps y with
// (h + pad - y) divisible by the stride, so the pixels with h mod stride_h = ph and w mod stride_w = pw form a class
// whose gradient is a UNIT-stride backward-data convolution of the same output gradient with the sub-sampled filter
// y = y0 + stride_h * j (the reference cuts the same classes into its kernel ids, backwardDataKernelIds,
// mlir/lib/Dialect/Rock/Transforms/loweringUtils.cpp:107-170). Each class runs through conv_run into a dense
// [n][h'][w'][g][c] block of the workspace, and this kernel interleaves the blocks into the caller's tensor. No
// product with a structural zero is computed, unlike the zero-upsampled formulation.
struct ClassTable {
  long long N, H, W, G, C;                 // the input gradient
  long long s_n, s_h, s_w, s_g, s_c;       // its strides in the caller's layout (elements)
  int sh, sw;
  long long off[16];                       // element offset of class ph * sw + pw inside the class area, -1: all zero
  int hs[16], wsz[16];                     // extents of the class block
};

template <int ES>
__global__ void interleave_classes_kernel(const uint8_t* __restrict__ cls, uint8_t* __restrict__ dst, ClassTable t) {
  // One thread per 16-byte vector of channels when the destination is channel-contiguous, else per element. One
  // block row of threads walks one image row (n, h): the class row, and with it every division by a run-time
  // extent, is computed once per row; along w the class alternates with w mod stride_w.
  const bool vec = t.s_c == 1 && (t.C * ES) % 16 == 0 && (t.s_n * ES) % 16 == 0 && (t.s_h * ES) % 16 == 0 &&
                   (t.s_w * ES) % 16 == 0 && (t.s_g * ES) % 16 == 0;
  const unsigned per = vec ? 16 / ES : 1;
  const unsigned cv = (unsigned)(t.C / per);
  const unsigned G = (unsigned)t.G, W = (unsigned)t.W, H = (unsigned)t.H;
  const unsigned row_items = W * G * cv;                       // < 2^31 (checked by the plan)
  const long long rows = t.N * t.H;
  if (row_items <= blockDim.x) {
    // the launch gave every item of a row its own thread: the position inside the row, and with it every division
    // but the two of the row index, is computed once
    if (threadIdx.x >= row_items) return;
    const unsigned i = threadIdx.x;
    const unsigned c = (i % cv) * per;
    const unsigned r = i / cv;
    const unsigned g = r % G, w = r / G;
    const unsigned kw = w % (unsigned)t.sw, wq = w / (unsigned)t.sw;
    const long long dcol = (long long)w * t.s_w + (long long)g * t.s_g + (long long)c * t.s_c;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
      const unsigned h = (unsigned)(row % H);
      const long long n = row / H;
      const unsigned k = (h % (unsigned)t.sh) * (unsigned)t.sw + kw, hq = h / (unsigned)t.sh;
      const long long d = n * t.s_n + (long long)h * t.s_h + dcol;
      const long long so = t.off[k] < 0 ? -1
                                        : t.off[k] + ((((n * t.hs[k] + hq) * t.wsz[k] + wq) * (long long)G + g) * t.C + c);
      if (vec) {
        *reinterpret_cast<uint4*>(dst + d * ES) = so < 0 ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(cls + so * ES);
      } else {
        if (ES == 2) reinterpret_cast<uint16_t*>(dst)[d] = so < 0 ? (uint16_t)0 : reinterpret_cast<const uint16_t*>(cls)[so];
        if (ES == 4) reinterpret_cast<uint32_t*>(dst)[d] = so < 0 ? 0u : reinterpret_cast<const uint32_t*>(cls)[so];
      }
    }
    return;
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const unsigned h = (unsigned)(row % H);
    const long long n = row / H;
    const unsigned ph = h % (unsigned)t.sh, hq = h / (unsigned)t.sh;
    const long long drow = n * t.s_n + (long long)h * t.s_h;
    for (unsigned i = threadIdx.x; i < row_items; i += blockDim.x) {
      const unsigned c = (i % cv) * per;
      const unsigned r = i / cv;
      const unsigned g = r % G, w = r / G;
      const unsigned k = ph * (unsigned)t.sw + w % (unsigned)t.sw, wq = w / (unsigned)t.sw;
      const long long d = drow + (long long)w * t.s_w + (long long)g * t.s_g + (long long)c * t.s_c;
      const long long so = t.off[k] < 0 ? -1
                                        : t.off[k] + ((((n * t.hs[k] + hq) * t.wsz[k] + wq) * (long long)G + g) * t.C + c);
      if (vec) {
        *reinterpret_cast<uint4*>(dst + d * ES) = so < 0 ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(cls + so * ES);
      } else {
        if (ES == 2) reinterpret_cast<uint16_t*>(dst)[d] = so < 0 ? (uint16_t)0 : reinterpret_cast<const uint16_t*>(cls)[so];
        if (ES == 4) reinterpret_cast<uint32_t*>(dst)[d] = so < 0 ? 0u : reinterpret_cast<const uint32_t*>(cls)[so];
      }
    }
  }
}

// The filter matrices of all stride classes in one pass. Class i gets B_i[c][(y', x', k)] =
// fil[k][c][y0 + stride_h * (ty - 1 - y')][x0 + stride_w * (tx - 1 - x')]: its sub-sampled taps, mirrored, in the
// c x (taps, k) form the unit-stride implicit GEMM reads (one group).
struct ClassFilters {
  long long s_k, s_c, s_y, s_x;     // filter strides in elements
  int K, C, sh, sw, n;
  int y0[16], x0[16], ty[16], tx[16];
  long long dst[16];                // element offset of B_i in the workspace
  long long first[17];              // prefix sums of the element counts
};

template <int ES>
__global__ void class_filters_kernel(const uint8_t* __restrict__ fil, uint8_t* __restrict__ ws, ClassFilters f) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < f.first[f.n]; i += (long long)gridDim.x * blockDim.x) {
    int c = 0;
    while (i >= f.first[c + 1]) ++c;
    unsigned r = (unsigned)(i - f.first[c]);            // a filter has far fewer than 2^32 elements
    const int k = (int)(r % (unsigned)f.K); r /= (unsigned)f.K;
    const int xp = (int)(r % (unsigned)f.tx[c]); r /= (unsigned)f.tx[c];
    const int yp = (int)(r % (unsigned)f.ty[c]);
    const int ch = (int)(r / (unsigned)f.ty[c]);
    const long long src = (long long)k * f.s_k + (long long)ch * f.s_c +
                          (long long)(f.y0[c] + f.sh * (f.ty[c] - 1 - yp)) * f.s_y +
                          (long long)(f.x0[c] + f.sw * (f.tx[c] - 1 - xp)) * f.s_x;
    const long long d = f.dst[c] + (i - f.first[c]);
    if (ES == 2) reinterpret_cast<uint16_t*>(ws)[d] = reinterpret_cast<const uint16_t*>(fil)[src];
    if (ES == 4) reinterpret_cast<uint32_t*>(ws)[d] = reinterpret_cast<const uint32_t*>(fil)[src];
  }
}

size_t up256(size_t x) { return (x + 255) / 256 * 256; }

// Named-dimension strides of a tensor stored in `layout` order (row-major over the letters).
bool layout_strides(const char* layout, const char* letters, const long long* sizes, long long* strides,
                    std::string* canon) {
  if (!layout || strlen(layout) != 5) return false;
  long long acc = 1;
  bool seen[5] = {false, false, false, false, false};
  for (int pos = 4; pos >= 0; --pos) {
    const char* f = strchr(letters, layout[pos]);
    if (!f) return false;
    const int idx = (int)(f - letters);
    if (seen[idx]) return false;
    seen[idx] = true;
    strides[idx] = acc;
    acc *= sizes[idx];
  }
  if (canon) *canon = layout;
  return true;
}

struct ConvPlan {
  // tensors: strides for fil (g,k,c,y,x), in (n,g,c,h,w), out (n,g,k,h,w)
  long long fs[5], is[5], os[5];
  RbGemmProblem gemm;
  // matrices: element counts (0 = operand used as it lies)
  bool a_direct, b_direct, c_direct;
  bool c_remap = false;   // forward, NKHW-like output: the GEMM epilogue stores channel-major per image (no transposing pass)
  bool a_implicit;   // forward: the A matrix is never built; the GEMM producer loads it from the NHWC input (TMA im2col)
  bool b_implicit;   // backward weight: the same for the B matrix (K = pixels, N = (y,x,c))
  bool a_up;         // backward data with a stride: the output gradient is zero-upsampled into the workspace first
  int a_planes;      // f32 forward implicit GEMM: TF32 planes of the input kept in the workspace (0, 1 or 2)
  bool a_nchw;       //   the input is NCHW: the plane pass transposes it to NHWC
  size_t a_bytes, b_bytes, c_bytes, gemm_ws;
  size_t a_off, b_off, c_off, gemm_off, total;
  // backward data by stride classes (see interleave_classes_kernel): sub-problems and their places in the workspace
  int n_classes = 0;
  struct StrideClass {
    RbConvProblem q;
    int ph, pw, y0, x0;
    size_t fil_off, out_off, ws_bytes;   // sub-filter, class block; out_off = SIZE_MAX for a class without taps
    RbGemmProblem gemm;                  // the class's GEMM when the whole set runs fused
    size_t gemm_ws;
    bool pointwise;                      //   a single tap without padding: A is the output gradient in place
  } cls[16];
  size_t cls_ws_off = 0;
  bool w_halo = false;      // backward weight on the halo kernel (csrc/conv_wgrad_halo_sm100.cu)
  HaloConv w_hc;
  bool cls_fused = false;   // every class takes the implicit unit-stride path: one filter pass, one GEMM per class
  bool fil_in_place = false;   // backward data on the halo kernel reads the KYXC filter as it lies (c contiguous)
  bool cls_halo = false;    //   ... and the halo kernel: up to four classes per launch, stored straight into the tensor
  bool cls_any_empty = false;
  HaloConv cls_hc[16];
};

bool is_dense_in_order(const long long* strides, const long long* sizes, const int* order, int n) {
  long long acc = 1;
  for (int i = n - 1; i >= 0; --i) {
    const int d = order[i];
    if (sizes[d] != 1 && strides[d] != acc) return false;
    acc *= sizes[d];
  }
  return true;
}

RbStatus make_plan(const RbConvProblem* p, ConvPlan* pl, int result_type = -1) {
  if (!p) return fail(RB_INVALID_PARAM, "problem is NULL");
  if (p->n <= 0 || p->g <= 0 || p->c <= 0 || p->k <= 0 || p->h <= 0 || p->w <= 0 || p->y <= 0 || p->x <= 0 ||
      p->stride_h <= 0 || p->stride_w <= 0 || p->dil_h <= 0 || p->dil_w <= 0 || p->pad_h < 0 || p->pad_w < 0 ||
      p->pad_h_r < 0 || p->pad_w_r < 0)
    return fail(RB_INVALID_PARAM, "convolution sizes must be positive (paddings non-negative)");
  if (p->direction < 0 || p->direction > 2) return fail(RB_INVALID_PARAM, "direction must be 0 (fwd), 1 (bwd data), 2 (bwd weight)");
  const long long ho = ((long long)p->h + p->pad_h + p->pad_h_r - (long long)(p->y - 1) * p->dil_h - 1) / p->stride_h + 1;
  const long long wo = ((long long)p->w + p->pad_w + p->pad_w_r - (long long)(p->x - 1) * p->dil_w - 1) / p->stride_w + 1;
  if (ho <= 0 || wo <= 0) return fail(RB_INVALID_PARAM, "the filter does not fit the padded image");
  if (p->ho != ho || p->wo != wo)
    return fail(RB_INVALID_PARAM, "ho/wo must equal (in + padL + padR - (fil-1)*dil - 1)/stride + 1 = " +
                                      std::to_string(ho) + " x " + std::to_string(wo));
  const int t = p->data_type;
  const bool f8 = t == RB_F8E4M3 || t == RB_F8E5M2;
  if (!(t == RB_F32 || t == RB_F16 || t == RB_BF16 || t == RB_I8 || f8)) return fail(RB_INVALID_PARAM, "unsupported element type");
  if ((t == RB_I8 || f8) && p->direction != 0)
    return fail(RB_UNSUPPORTED, "8-bit convolutions exist in the forward direction only (RockOps.td:101-134, ConvGenerator.cpp:631-638)");
  const long long fsz[5] = {p->g, p->k, p->c, p->y, p->x};
  const long long isz[5] = {p->n, p->g, p->c, p->h, p->w};
  const long long osz[5] = {p->n, p->g, p->k, ho, wo};
  if (!layout_strides(p->fil_layout, "gkcyx", fsz, pl->fs, nullptr)) return fail(RB_INVALID_PARAM, "fil_layout must be a permutation of gkcyx");
  if (!layout_strides(p->in_layout, "ngchw", isz, pl->is, nullptr)) return fail(RB_INVALID_PARAM, "in_layout must be a permutation of ngchw");
  if (!layout_strides(p->out_layout, "ngkhw", osz, pl->os, nullptr)) return fail(RB_INVALID_PARAM, "out_layout must be a permutation of ngkhw");

  const size_t es = dtype_bytes(t);
  // rocmlir-gen: -t i8 => i32 output, 8-bit floats => f32; a fused epilogue of the forward direction may declare
  // another result type (quant_convolution -> dequantize -> quantize ends in i8)
  const int out_t = (p->direction == 0 && result_type >= 0) ? result_type : (t == RB_I8) ? RB_I32 : f8 ? RB_F32 : t;
  const size_t es_o = dtype_bytes(out_t);
  const long long G = p->g;
  const long long pix_o = (long long)p->n * ho * wo, pix_i = (long long)p->n * p->h * p->w;
  const long long yxc = (long long)p->y * p->x * p->c, yxk = (long long)p->y * p->x * p->k;
  const bool pointwise = p->y == 1 && p->x == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_h == 0 &&
                         p->pad_w == 0 && p->pad_h_r == 0 && p->pad_w_r == 0;
  RbGemmProblem& gp = pl->gemm;
  memset(&gp, 0, sizeof(gp));
  pl->a_implicit = false;
  pl->b_implicit = false;
  pl->a_up = false;
  pl->a_planes = 0;
  pl->a_nchw = false;
  gp.g = (int)G;
  gp.ab_type = t;
  gp.f32_mode = p->f32_mode;
  // dense-order tests: index orders into (n,g,c/k,h,w) and (g,k,c,y,x)
  const int act_gmat[5] = {1, 0, 3, 4, 2};   // g, n, h, w, c : the [G][pixels][channels] matrix order
  const int fil_kyxc[5] = {0, 1, 3, 4, 2};   // g, k, y, x, c : the [G][k][(y,x,c)] matrix order
  const bool in_is_mat = is_dense_in_order(pl->is, isz, act_gmat, 5);
  const bool out_is_mat = is_dense_in_order(pl->os, osz, act_gmat, 5);
  const bool fil_is_mat = is_dense_in_order(pl->fs, fsz, fil_kyxc, 5);
  if (p->direction == 0) {
    gp.m = (int)pix_o; gp.n = p->k; gp.k = (int)yxc;
    gp.trans_a = 0; gp.trans_b = 1; gp.trans_c = 0;       // A [M][K], B [N][K], C [M][N]
    gp.c_type = out_t;
    pl->a_direct = pointwise && in_is_mat;
    pl->b_direct = fil_is_mat;
    pl->c_direct = out_is_mat;
    // NHWC input, one group, channels a multiple of the 128-byte K block, 8/16-bit types: implicit GEMM.
    // Corner / offset fields of the im2col descriptor are small signed integers; stay well inside them.
    // f32: the same over TF32 planes of the input (hi, and lo in accurate mode) in NHWC order, built by one pass
    // over the input - a transposing pass when the input is NCHW - instead of an im2col matrix Y*X times its size.
    const int act_nchw[5] = {0, 1, 2, 3, 4};
    const bool in_is_nchw = is_dense_in_order(pl->is, isz, act_nchw, 5);
    const bool in_ok = (t != RB_F32) ? in_is_mat : (in_is_mat || in_is_nchw);
    pl->a_implicit = !pl->a_direct && in_ok && G == 1 && (p->c * es) % 128 == 0 &&
                     p->pad_h < 64 && p->pad_w < 64 && (p->y - 1) * p->dil_h < 256 && (p->x - 1) * p->dil_w < 256 &&
                     p->stride_h <= 8 && p->stride_w <= 8 && pix_i < 0x7fffffffLL;
    pl->a_planes = 0;
    pl->a_nchw = false;
    if (pl->a_implicit && t == RB_F32) {
      pl->a_nchw = !in_is_mat;
      pl->a_planes = p->f32_mode == 0 ? 2 : (in_is_mat ? 0 : 1);
    }
    if (pl->a_implicit) pl->a_direct = true;   // nothing to gather
    pl->a_bytes = pl->a_implicit ? (size_t)pl->a_planes * up256((size_t)pix_i * p->c * es)
                                 : (pl->a_direct ? 0 : (size_t)G * pix_o * yxc * es);
    pl->b_bytes = pl->b_direct ? 0 : (size_t)G * p->k * yxc * es;
    pl->c_bytes = pl->c_direct ? 0 : (size_t)G * pix_o * p->k * es_o;
  } else if (p->direction == 2) {
    gp.m = p->k; gp.n = (int)yxc; gp.k = (int)pix_o;
    gp.trans_a = 1; gp.trans_b = 0; gp.trans_c = 0;       // A stored [K][M] = out matrix, B [K][N] = im2col, C [M][N]
    gp.c_type = t;
    pl->a_direct = out_is_mat;
    pl->b_direct = pointwise && in_is_mat;
    pl->c_direct = fil_is_mat;
    // NHWC input, one group, 16-bit types: the im2col matrix is never built; the producer fetches its tiles from the
    // input tensor (one im2col load per 64-channel chunk of a tile, K index = output pixel)
    pl->b_implicit = !pl->b_direct && in_is_mat && G == 1 && t != RB_F32 && (p->c * es) % 128 == 0 &&
                     p->pad_h < 64 && p->pad_w < 64 && (p->y - 1) * p->dil_h < 256 && (p->x - 1) * p->dil_w < 256 &&
                     p->stride_h <= 8 && p->stride_w <= 8;
    if (pl->b_implicit) pl->b_direct = true;
    // unit stride, dense NHWK output gradient and KYXC filter gradient: the halo form (input window loaded once per tile)
    pl->w_halo = false;
    if (pl->b_implicit && pl->a_direct && pl->c_direct && p->stride_h == 1 && p->stride_w == 1) {
      HaloConv& h = pl->w_hc;
      h.is_bf16 = t == RB_BF16;
      h.N = p->n; h.H = p->h; h.W = p->w; h.C = p->c; h.P = (int)ho; h.Q = (int)wo; h.Kout = p->k;
      h.Y = p->y; h.X = p->x; h.dil_h = p->dil_h; h.dil_w = p->dil_w;
      h.pad_h = p->pad_h; h.pad_w = p->pad_w; h.pad_h_r = p->pad_h_r; h.pad_w_r = p->pad_w_r;
      h.o_n = h.o_p = h.o_q = 0;
      pl->w_halo = conv_wgrad_halo_applicable(h);
    }
    pl->a_bytes = pl->a_direct ? 0 : (size_t)G * pix_o * p->k * es;
    pl->b_bytes = pl->b_direct ? 0 : (size_t)G * pix_o * yxc * es;
    pl->c_bytes = pl->c_direct ? 0 : (size_t)G * p->k * yxc * es;
  } else {
    gp.m = (int)pix_i; gp.n = p->c; gp.k = (int)yxk;
    gp.trans_a = 0; gp.trans_b = 0; gp.trans_c = 0;       // A [M][K] = col2im(out), B [K][N] = filter as (y,x,k) x c
    gp.c_type = result_type >= 0 ? result_type : t;
    if (result_type >= 0 && !in_is_mat)
      return fail(RB_UNSUPPORTED, "a widened input gradient needs the [pixels][channels] input layout");
    pl->a_direct = pointwise && out_is_mat;
    // a 1x1 filter stored (g,k,c) row-major already is the [K][N] matrix
    const int fil_yxkc[5] = {0, 3, 4, 1, 2};
    pl->b_direct = is_dense_in_order(pl->fs, fsz, fil_yxkc, 5);
    pl->c_direct = in_is_mat;
    // Unit stride: the input gradient is a forward convolution of the output gradient with the filter taps
    // mirrored, so the same implicit-GEMM path applies (A = NHWK output gradient read through im2col loads with
    // padding (fil-1)*dil - pad; B = the filter rearranged to c x (y', x', k) with y' = Y-1-y, x' = X-1-x).
    const long long bpad_h = (long long)(p->y - 1) * p->dil_h - p->pad_h, bpad_w = (long long)(p->x - 1) * p->dil_w - p->pad_w;
    // A stride is handled by zero-upsampling the output gradient first ((Ho-1)*stride+1 rows with the gradient on
    // every stride-th position): the same unit-stride formulation then applies. It computes stride_h*stride_w times
    // the useful products, and still beats the col2im gather it replaces.
    const long long uh = (ho - 1) * p->stride_h + 1, uw = (wo - 1) * p->stride_w + 1;
    const long long bpad_h_hi = p->h - uh - bpad_h + (long long)(p->y - 1) * p->dil_h;
    const long long bpad_w_hi = p->w - uw - bpad_w + (long long)(p->x - 1) * p->dil_w;
    pl->a_up = p->stride_h > 1 || p->stride_w > 1;
    pl->a_implicit = (!pl->a_direct || pl->a_up) && out_is_mat && G == 1 && t != RB_F32 && (p->k * es) % 128 == 0 &&
                     bpad_h >= 0 && bpad_w >= 0 && bpad_h < 64 && bpad_w < 64 && bpad_h_hi >= 0 && bpad_w_hi >= 0 &&
                     bpad_h_hi < 64 && bpad_w_hi < 64 && p->stride_h <= 4 && p->stride_w <= 4 &&
                     (p->y - 1) * p->dil_h < 256 && (p->x - 1) * p->dil_w < 256 &&
                     (long long)p->n * uh * uw < 0x7fffffffLL;
    if (!pl->a_implicit) pl->a_up = false;
    if (pl->a_implicit) {
      pl->a_direct = true;
      pl->b_direct = false;     // the mirrored c x (y',x',k) matrix is always built (it is filter-sized)
      gp.trans_b = 1;           // B stored [N = c][K = (y',x',k)]
    }
    pl->a_bytes = pl->a_up ? (size_t)p->n * uh * uw * p->k * es : (pl->a_direct ? 0 : (size_t)G * pix_i * yxk * es);
    pl->b_bytes = pl->b_direct ? 0 : (size_t)G * yxk * p->c * es;
    pl->c_bytes = pl->c_direct ? 0 : (size_t)G * pix_i * p->c * es;
  }
  if ((long long)gp.m != (p->direction == 0 ? pix_o : p->direction == 2 ? (long long)p->k : pix_i) ||
      pix_o > 0x7fffffffLL || pix_i > 0x7fffffffLL || yxc > 0x7fffffffLL || yxk > 0x7fffffffLL)
    return fail(RB_UNSUPPORTED, "GEMM extent exceeds 2^31");
  pl->n_classes = 0;
  if (p->direction == 1 && result_type < 0 && (p->stride_h > 1 || p->stride_w > 1) && p->dil_h == 1 && p->dil_w == 1 &&
      p->stride_h <= 4 && p->stride_w <= 4) {
    // stride classes: every class is a unit-stride backward-data problem over the same output gradient
    bool ok = true, fused = true;
    size_t off = 0, sub_ws = 0;
    int nc = 0;
    for (int ph = 0; ph < p->stride_h && ok; ++ph)
      for (int pw = 0; pw < p->stride_w && ok; ++pw) {
        ConvPlan::StrideClass& c = pl->cls[nc++];
        memset(&c.q, 0, sizeof(c.q));
        c.ph = ph; c.pw = pw;
        const int hs = (p->h - ph + p->stride_h - 1) / p->stride_h, wsz = (p->w - pw + p->stride_w - 1) / p->stride_w;
        c.y0 = (ph + p->pad_h) % p->stride_h; c.x0 = (pw + p->pad_w) % p->stride_w;
        const int ty = c.y0 < p->y ? (p->y - c.y0 + p->stride_h - 1) / p->stride_h : 0;
        const int tx = c.x0 < p->x ? (p->x - c.x0 + p->stride_w - 1) / p->stride_w : 0;
        const int q0h = (ph + p->pad_h) / p->stride_h, q0w = (pw + p->pad_w) / p->stride_w;
        c.q.n = p->n; c.q.g = p->g; c.q.c = p->c; c.q.k = p->k;
        c.q.h = hs; c.q.w = wsz; c.q.y = ty; c.q.x = tx;
        c.q.stride_h = c.q.stride_w = c.q.dil_h = c.q.dil_w = 1;
        c.q.pad_h = q0h; c.q.pad_w = q0w;
        c.q.pad_h_r = (int)ho - hs - q0h + ty - 1; c.q.pad_w_r = (int)wo - wsz - q0w + tx - 1;
        c.q.ho = (int)ho; c.q.wo = (int)wo;
        c.q.data_type = t; c.q.direction = 1; c.q.f32_mode = p->f32_mode;
        strcpy(c.q.fil_layout, "gkyxc");
        strcpy(c.q.in_layout, "nhwgc");
        memcpy(c.q.out_layout, p->out_layout, sizeof(c.q.out_layout));
        c.fil_off = c.out_off = 0; c.ws_bytes = 0;
        if (hs <= 0 || wsz <= 0) { ok = false; break; }       // fewer input pixels than the stride: not worth a path
        if (ty == 0 || tx == 0) { c.out_off = SIZE_MAX; continue; }   // no tap reaches this class: zeros
        if (c.q.pad_h_r < 0 || c.q.pad_w_r < 0) { ok = false; break; }
        c.fil_off = off; off += up256((size_t)G * p->k * ty * tx * p->c * es);
        c.out_off = off; off += up256((size_t)p->n * hs * wsz * G * p->c * es);
        {
          ConvPlan sub;
          if (make_plan(&c.q, &sub, -1) != RB_SUCCESS) { ok = false; break; }
          c.ws_bytes = sub.total;
          c.gemm = sub.gemm;
          c.gemm_ws = sub.gemm_ws;
          c.pointwise = !sub.a_implicit && sub.a_direct;   // one tap, no padding: the output gradient is the A matrix
          if (c.pointwise) {
            c.gemm.trans_b = 1;                            // the filter pass writes c x k for every class
            c.gemm_ws = gemm_workspace_bytes(&c.gemm, -1);
          }
          if (!((sub.a_implicit || c.pointwise) && sub.c_direct && !sub.a_up && G == 1)) fused = false;
        }
        sub_ws = std::max(sub_ws, c.ws_bytes);
      }
    if (ok) {
      pl->cls_fused = fused;
      pl->n_classes = nc;
      // Every class is a unit-stride convolution of the output gradient: on the halo kernel each one writes its pixels
      // straight into the caller's tensor (pixel strides = the convolution's strides), so the class blocks in the
      // workspace and the interleaving pass fall away.
      pl->cls_halo = fused && pl->c_direct && es == 2;
      pl->cls_any_empty = false;
      for (int i = 0; i < nc && pl->cls_halo; ++i) {
        const ConvPlan::StrideClass& c = pl->cls[i];
        if (c.out_off == SIZE_MAX) { pl->cls_any_empty = true; continue; }
        HaloConv& h = pl->cls_hc[i];
        h.is_bf16 = p->data_type == RB_BF16;
        h.N = p->n; h.H = (int)ho; h.W = (int)wo; h.C = p->k; h.P = c.q.h; h.Q = c.q.w; h.Kout = p->c;
        h.Y = c.q.y; h.X = c.q.x; h.dil_h = h.dil_w = 1;
        h.pad_h = (c.q.y - 1) - c.q.pad_h; h.pad_w = (c.q.x - 1) - c.q.pad_w;
        h.pad_h_r = c.q.h - (int)ho - h.pad_h + (c.q.y - 1); h.pad_w_r = c.q.w - (int)wo - h.pad_w + (c.q.x - 1);
        h.o_q = (long long)p->stride_w * p->c; h.o_p = (long long)p->stride_h * p->w * p->c; h.o_n = (long long)p->h * p->w * p->c;
        if (pl->fs[2] == 1 && G == 1 && p->c % 64 == 0) {   // taps come straight from the filter tensor
          h.b_mn = true;
          h.FY = p->y; h.FX = p->x; h.f_sk = pl->fs[1]; h.f_sy = pl->fs[3]; h.f_sx = pl->fs[4];
          h.fy0 = c.y0; h.fsy = p->stride_h; h.fx0 = c.x0; h.fsx = p->stride_w;
          if (!conv_halo_applicable(h)) h.b_mn = false;
        }
        pl->cls_halo = conv_halo_applicable(h);
      }
      pl->fil_in_place = pl->cls_halo;
      for (int i = 0; i < nc && pl->cls_halo; ++i)
        if (pl->cls[i].out_off != SIZE_MAX && !pl->cls_hc[i].b_mn) pl->fil_in_place = false;
      if (!pl->fil_in_place)
        for (int i = 0; i < nc; ++i) pl->cls_hc[i].b_mn = false;
      pl->cls_ws_off = off;
      pl->total = off + up256(sub_ws);
      pl->gemm_ws = 0;
      return RB_SUCCESS;
    }
  }
  pl->c_remap = false;
  if (p->direction == 0 && !pl->c_direct && pl->a_implicit && G == 1 && pl->os[4] == 1 && pl->os[3] == wo &&
      pl->os[2] == ho * wo && pl->os[0] == (long long)p->k * ho * wo) {
    RbGemmConfigInfo info;
    if (rbGemmGetConfig(&gp, &info) == RB_SUCCESS && info.splits == 1) {
      pl->c_remap = true;
      pl->c_bytes = 0;
    }
  }
  pl->gemm_ws = gemm_workspace_bytes(&gp, pl->a_implicit ? 0 : pl->b_implicit ? 1 : -1);
  if (p->direction == 2 && pl->w_halo) pl->gemm_ws = std::max(pl->gemm_ws, conv_wgrad_halo_workspace(pl->w_hc));
  size_t off = 0;
  pl->a_off = off; off += up256(pl->a_bytes);
  pl->b_off = off; off += up256(pl->b_bytes);
  pl->c_off = off; off += up256(pl->c_bytes);
  pl->gemm_off = off; off += up256(pl->gemm_ws);
  pl->total = off;
  return RB_SUCCESS;
}

template <typename K, typename... Args>
void launch_es(size_t es, int blocks, cudaStream_t st, K k1, K k2, K k4, Args... args) {
  if (es == 1) k1<<<blocks, 256, 0, st>>>(args...);
  else if (es == 2) k2<<<blocks, 256, 0, st>>>(args...);
  else k4<<<blocks, 256, 0, st>>>(args...);
}

}  // namespace
}  // namespace rb

using namespace rb;

// Unit-stride 16-bit NHWC forward / backward-data convolutions whose filter fits into shared memory run on the halo
// kernel: the window of an output tile is loaded once instead of once per tap (csrc/conv_halo_sm100.cu). Backward
// data is the same kernel over the output gradient with mirrored taps, which it reads straight from a KYXC filter
// (hc->b_mn) when the layout allows. Variant bit 26 keeps the im2col form.
static void halo_geometry(const RbConvProblem* p, HaloConv* hc);
static bool f32_streamed(const RbConvProblem* p, const ConvPlan& pl, HaloConv* sc, long long* o_k);
static bool filter_is_kcyx(const RbConvProblem* p, const ConvPlan& pl);
static bool unit_halo(const RbConvProblem* p, const ConvPlan& pl, bool has_epi, HaloConv* hc) {
  if (p->direction > 1 || !pl.a_implicit || pl.a_planes != 0 || pl.a_up || !pl.c_direct || p->stride_h != 1 || p->stride_w != 1 ||
      !(p->data_type == RB_F16 || p->data_type == RB_BF16) || !(has_epi || pl.gemm.c_type == p->data_type) ||
      ((rbGetGemmVariant() >> 26) & 1))
    return false;
  halo_geometry(p, hc);
  if (p->direction == 1 && pl.fs[2] == 1 && p->g == 1 && p->c % 64 == 0) {
    hc->b_mn = true;
    hc->FY = p->y; hc->FX = p->x; hc->f_sk = pl.fs[1]; hc->f_sy = pl.fs[3]; hc->f_sx = pl.fs[4];
    hc->fy0 = 0; hc->fsy = 1; hc->fx0 = 0; hc->fsx = 1;
    if (conv_halo_applicable(*hc)) return true;
    hc->b_mn = false;
  }
  return conv_halo_applicable(*hc);
}

// f32 forward on the streamed-filter halo kernel (csrc/conv_halo_stream_sm100.cu): unit stride, one group, the image as
// two TF32 planes; the kernel stores the result with the output tensor's own strides (NHWK, NKHW or any other order).
static bool f32_streamed(const RbConvProblem* p, const ConvPlan& pl, HaloConv* sc, long long* o_k) {
  const size_t fil_plane = up256((size_t)p->k * p->y * p->x * p->c * 4);
  if (!(pl.a_implicit && !pl.a_up && p->direction == 0 && p->stride_h == 1 && p->stride_w == 1 && p->g == 1 &&
        !((rbGetGemmVariant() >> 26) & 1) && p->data_type == RB_F32 && pl.a_planes == 2 && pl.gemm.c_type == RB_F32 &&
        pl.gemm_ws >= 2 * fil_plane))
    return false;
  halo_geometry(p, sc);
  *o_k = 1;
  if (!pl.c_direct) { sc->o_n = pl.os[0]; sc->o_p = pl.os[3]; sc->o_q = pl.os[4]; *o_k = pl.os[2]; }
  return conv_halo_stream_applicable(*sc, 4, *o_k);
}
static bool filter_is_kcyx(const RbConvProblem* p, const ConvPlan& pl) {
  return p->g == 1 && pl.fs[4] == 1 && pl.fs[3] == p->x && pl.fs[2] == (long long)p->y * p->x &&
         pl.fs[1] == (long long)p->c * p->y * p->x;
}

// The unit-stride convolution as the halo kernels see it: forward over the input, or backward data as a forward
// convolution of the output gradient (channels-last result with dense pixel strides).
static void halo_geometry(const RbConvProblem* p, HaloConv* hc) {
  const int ho = p->ho, wo = p->wo;
  hc->is_bf16 = p->data_type == RB_BF16;
  hc->Y = p->y; hc->X = p->x; hc->dil_h = p->dil_h; hc->dil_w = p->dil_w;
  if (p->direction == 0) {
    hc->N = p->n; hc->H = p->h; hc->W = p->w; hc->C = p->c; hc->P = ho; hc->Q = wo; hc->Kout = p->k;
    hc->pad_h = p->pad_h; hc->pad_w = p->pad_w; hc->pad_h_r = p->pad_h_r; hc->pad_w_r = p->pad_w_r;
  } else {   // backward data: a forward convolution of the output gradient with the mirrored filter
    hc->N = p->n; hc->H = ho; hc->W = wo; hc->C = p->k; hc->P = p->h; hc->Q = p->w; hc->Kout = p->c;
    hc->pad_h = (p->y - 1) * p->dil_h - p->pad_h; hc->pad_w = (p->x - 1) * p->dil_w - p->pad_w;
    hc->pad_h_r = p->h - ho - hc->pad_h + (p->y - 1) * p->dil_h; hc->pad_w_r = p->w - wo - hc->pad_w + (p->x - 1) * p->dil_w;
  }
  hc->o_q = hc->Kout; hc->o_p = (long long)hc->Q * hc->Kout; hc->o_n = (long long)hc->P * hc->Q * hc->Kout;
}

size_t rb::conv_workspace_bytes(const RbConvProblem* p, int result_type) {
  TunedVariantScope tuned(tuned_variant_conv(p));
  ConvPlan pl;
  if (make_plan(p, &pl, result_type) != RB_SUCCESS) return 0;
  return pl.total;
}

extern "C" size_t rbConvWorkspaceSize(const RbConvProblem* p) { return rb::conv_workspace_bytes(p, -1); }

extern "C" RbStatus rbConvGetGemmProblem(const RbConvProblem* p, RbGemmProblem* out) {
  ConvPlan pl;
  RbStatus st = make_plan(p, &pl);
  if (st != RB_SUCCESS) return st;
  if (!out) return fail(RB_INVALID_PARAM, "out is NULL");
  *out = pl.gemm;
  return RB_SUCCESS;
}

extern "C" int rbConvKernelCount(const RbConvProblem* p) {
  TunedVariantScope tuned(tuned_variant_conv(p));
  ConvPlan pl;
  if (make_plan(p, &pl) != RB_SUCCESS) return -1;
  const bool halo_off = ((rbGetGemmVariant() >> 26) & 1) != 0;
  if (pl.n_classes > 0 && pl.cls_halo && !halo_off) {
    int live = 0;
    for (int i = 0; i < pl.n_classes; ++i) live += pl.cls[i].out_off != SIZE_MAX;
    return (pl.fil_in_place ? 0 : 1) + (live + 3) / 4 + (pl.cls_any_empty ? 1 : 0);   // filter pass (unless the filter is read in place), four classes per launch, zero fill
  }
  if (p->direction == 2 && pl.w_halo && !halo_off) return 2;   // weight-gradient kernel + the sum of its slabs
  {
    HaloConv hc;
    if (pl.n_classes == 0 && unit_halo(p, pl, false, &hc) && hc.b_mn) return 1;   // backward data, filter read in place
  }
  {
    HaloConv sc;
    long long o_k;
    if (pl.n_classes == 0 && f32_streamed(p, pl, &sc, &o_k))   // image planes, filter planes (after a permutation unless KYXC / KCYX), kernel
      return 3 + ((pl.b_direct || filter_is_kcyx(p, pl)) ? 0 : 1);
  }
  if (pl.n_classes > 0) {
    int n = 1 + (pl.cls_fused ? 1 : 0);   // the interleaving pass (and the one filter pass of the fused form)
    for (int i = 0; i < pl.n_classes; ++i)
      if (pl.cls[i].out_off != SIZE_MAX) n += pl.cls_fused ? 1 : 1 + rbConvKernelCount(&pl.cls[i].q);
    return n;
  }
  return 1 + (pl.a_direct ? 0 : 1) + (pl.b_direct ? 0 : 1) + ((pl.c_direct || pl.c_remap) ? 0 : 1);
}

extern "C" RbStatus rbConv(const RbConvProblem* p, void* filter, void* input, void* output, void* workspace,
                           size_t workspace_bytes, void* stream_v) {
  return rb::conv_run(p, -1, filter, input, output, workspace, workspace_bytes, stream_v);
}

extern "C" size_t rbConvEpiWorkspaceSize(const RbConvProblem* p, int32_t out_type) {
  return rb::conv_workspace_bytes(p, out_type);
}

extern "C" RbStatus rbConvEpi(const RbConvProblem* p, const RbEpilogue* epi, int32_t out_type, void* filter, void* input,
                              void* output, void* workspace, size_t workspace_bytes, void* stream_v) {
  if (p && p->direction != 0) return fail(RB_UNSUPPORTED, "a fused epilogue exists for the forward convolution only");
  if (out_type >= 0 && !dtype_bytes(out_type)) return fail(RB_INVALID_PARAM, "unknown out_type");
  return rb::conv_run(p, out_type, filter, input, output, workspace, workspace_bytes, stream_v, epi);
}

extern "C" RbStatus rbConvEncodeLaunch(const RbConvProblem* p, const RbEpilogue* epi, int32_t out_type, void* filter,
                                       void* input, void* output, RbKernelLaunch* out) {
  if (!out) return fail(RB_INVALID_PARAM, "out is NULL");
  return rb::conv_run(p, out_type, filter, input, output, nullptr, 0, nullptr, epi, out);
}

RbStatus rb::conv_run(const RbConvProblem* p, int result_type, void* filter, void* input, void* output, void* workspace,
                      size_t workspace_bytes, void* stream_v, const RbEpilogue* epi, RbKernelLaunch* capture) {
  TunedVariantScope tuned(tuned_variant_conv(p));
  ConvPlan pl;
  RbStatus st = make_plan(p, &pl, result_type);
  if (st != RB_SUCCESS) return st;
  if (capture && (pl.n_classes > 0 || !pl.a_direct || !pl.b_direct || !pl.c_direct || pl.a_up || pl.a_planes > 0 ||
                  (p->direction == 1 && pl.a_implicit)))
    return fail(RB_UNSUPPORTED, "this convolution runs as several kernels (layout, filter or reduction passes): it has no "
                                "single-kernel binary; launch it through the library");
  if (epi && p->direction != 0) return fail(RB_UNSUPPORTED, "a fused epilogue exists for the forward convolution only");
  if (epi && (epi->flags & RB_EPI_RESIDUAL) && !pl.c_direct)
    return fail(RB_UNSUPPORTED, "a residual operand needs the [pixels][channels] output layout (nhwgk)");
  if (epi && (epi->flags & RB_EPI_BIAS_ROW)) return fail(RB_UNSUPPORTED, "the bias of a convolution is per output channel or scalar");
  if (!filter || !input || !output) return fail(RB_INVALID_PARAM, "filter, input and output must be device pointers");
  if (!capture && pl.total > 0 && (!workspace || workspace_bytes < pl.total))
    return fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(pl.total) + " bytes required");
  const DeviceInfo* dev = device_info();
  if (!dev) return RB_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const size_t es = dtype_bytes(p->data_type);
  const int blocks = dev->sm_count * 8;
  const long long ho = p->ho, wo = p->wo;

  auto gather = [&](const void* src, uint8_t* dst, bool from_out, bool transposed, long long P, long long Q,
                    long long CH) {
    GatherParams g;
    g.N = p->n; g.G = p->g; g.P = P; g.Q = Q; g.Y = p->y; g.X = p->x; g.CH = CH;
    g.pitch = g.Y * g.X * g.CH;
    const long long* s = from_out ? pl.os : pl.is;
    g.s_n = s[0]; g.s_g = s[1]; g.s_ch = s[2]; g.s_a = s[3]; g.s_b = s[4];
    g.A = from_out ? ho : p->h; g.B = from_out ? wo : p->w;
    g.stride_h = p->stride_h; g.stride_w = p->stride_w; g.dil_h = p->dil_h; g.dil_w = p->dil_w;
    g.pad_h = p->pad_h; g.pad_w = p->pad_w;
    g.transposed = transposed ? 1 : 0;
    const bool vec = g.s_ch == 1 && (g.CH * (long long)es) % 16 == 0 && (g.pitch * (long long)es) % 16 == 0 &&
                     (g.s_n * (long long)es) % 16 == 0 && (g.s_g * (long long)es) % 16 == 0 &&
                     (g.s_a * (long long)es) % 16 == 0 && (g.s_b * (long long)es) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                     g.N * g.P * g.Q < 0x7fffffffLL && g.pitch < 0x7fffffffLL;
    if (vec)
      launch_es(es, blocks, stream, conv_gather_vec_kernel<1>, conv_gather_vec_kernel<2>, conv_gather_vec_kernel<4>,
                static_cast<const uint8_t*>(src), dst, g);
    else
      launch_es(es, blocks, stream, conv_gather_kernel<1>, conv_gather_kernel<2>, conv_gather_kernel<4>,
                static_cast<const uint8_t*>(src), dst, g);
    count_launch();
  };
  auto permute = [&](const void* src, void* dst, const long long* sizes, const long long* strides, const int* order,
                     bool to_dense, size_t esz) {
    Dims5 d;
    for (int i = 0; i < 5; ++i) { d.size[i] = sizes[order[i]]; d.stride[i] = strides[order[i]]; }
    // dense (b0, b1, r_hi, r_lo, c) against a tensor whose (r_hi, r_lo) run is contiguous: batched 2-D transpose
    if (d.stride[3] == 1 && d.stride[2] == d.size[3] && d.size[4] >= 8 && d.size[2] * d.size[3] >= 32 &&
        d.stride[0] >= 0 && d.stride[1] >= 0 && d.stride[4] > 0) {
      Transpose2 t;
      t.B0 = d.size[0]; t.B1 = d.size[1]; t.R = d.size[2] * d.size[3]; t.C = d.size[4];
      t.s_b0 = d.stride[0]; t.s_b1 = d.stride[1]; t.s_c = d.stride[4];
      const long long tiles = t.B0 * t.B1 * ((t.R + 31) / 32) * ((t.C + 31) / 32);
      const int tb = (int)std::min<long long>(tiles, (long long)dev->sm_count * 16);
      const int td = to_dense ? 1 : 0;
      if (esz == 1)
        transpose_tiles_kernel<uint8_t><<<tb, 256, 0, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), t, td);
      else if (esz == 2)
        transpose_tiles_kernel<uint16_t><<<tb, 256, 0, stream>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), t, td);
      else
        transpose_tiles_kernel<uint32_t><<<tb, 256, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), t, td);
      count_launch();
      return;
    }
    const long long elems = d.size[0] * d.size[1] * d.size[2] * d.size[3] * d.size[4];
    const int pb = (int)std::max<long long>(1, std::min<long long>(blocks, (elems + 1023) / 1024));   // filters are small
    launch_es(esz, pb, stream, permute5_kernel<1>, permute5_kernel<2>, permute5_kernel<4>,
              static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), d, to_dense ? 1 : 0);
    count_launch();
  };
  const long long fsz[5] = {p->g, p->k, p->c, p->y, p->x};
  const long long isz[5] = {p->n, p->g, p->c, p->h, p->w};
  const long long osz[5] = {p->n, p->g, p->k, ho, wo};
  const int act_gmat[5] = {1, 0, 3, 4, 2};
  const int fil_kyxc[5] = {0, 1, 3, 4, 2};
  const int fil_yxkc[5] = {0, 3, 4, 1, 2};
  const size_t es_c = dtype_bytes(pl.gemm.c_type);

  if (pl.n_classes > 0) {
    ClassTable tb;
    tb.N = p->n; tb.H = p->h; tb.W = p->w; tb.G = p->g; tb.C = p->c;
    tb.s_n = pl.is[0]; tb.s_g = pl.is[1]; tb.s_c = pl.is[2]; tb.s_h = pl.is[3]; tb.s_w = pl.is[4];
    tb.sh = p->stride_h; tb.sw = p->stride_w;
    for (int i = 0; i < 16; ++i) { tb.off[i] = -1; tb.hs[i] = tb.wsz[i] = 1; }
    const bool cls_on_halo = pl.cls_halo && !((rbGetGemmVariant() >> 26) & 1);
    if (pl.cls_fused && !(cls_on_halo && pl.fil_in_place)) {
      ClassFilters ft;
      ft.s_k = pl.fs[1]; ft.s_c = pl.fs[2]; ft.s_y = pl.fs[3]; ft.s_x = pl.fs[4];
      ft.K = p->k; ft.C = p->c; ft.sh = p->stride_h; ft.sw = p->stride_w;
      ft.n = 0;
      ft.first[0] = 0;
      for (int i = 0; i < pl.n_classes; ++i) {
        const ConvPlan::StrideClass& c = pl.cls[i];
        if (c.out_off == SIZE_MAX) continue;
        const int j = ft.n++;
        ft.y0[j] = c.y0; ft.x0[j] = c.x0; ft.ty[j] = c.q.y; ft.tx[j] = c.q.x;
        ft.dst[j] = (long long)(c.fil_off / es);
        ft.first[j + 1] = ft.first[j] + (long long)p->c * c.q.y * c.q.x * p->k;
      }
      const int fb = (int)std::max<long long>(1, std::min<long long>(blocks, (ft.first[ft.n] + 1023) / 1024));
      if (es == 2) class_filters_kernel<2><<<fb, 256, 0, stream>>>(static_cast<const uint8_t*>(filter), ws, ft);
      else class_filters_kernel<4><<<fb, 256, 0, stream>>>(static_cast<const uint8_t*>(filter), ws, ft);
      count_launch();
    }
    if (cls_on_halo) {
      if (pl.cls_any_empty) {   // pixels no tap reaches
        RB_CUDA_TRY(cudaMemsetAsync(input, 0, (size_t)p->n * p->h * p->w * p->c * es, stream));
        count_launch();
      }
      // four classes per launch (a 2 x 2 stride has exactly four)
      HaloConv group[4];
      const void* fils[4];
      void* firsts[4];
      int n = 0;
      for (int i = 0; i <= pl.n_classes; ++i) {
        if (i < pl.n_classes && pl.cls[i].out_off != SIZE_MAX) {
          const ConvPlan::StrideClass& c = pl.cls[i];
          group[n] = pl.cls_hc[i];
          fils[n] = pl.fil_in_place ? static_cast<const void*>(filter) : static_cast<const void*>(ws + c.fil_off);
          firsts[n] = static_cast<uint8_t*>(input) + ((size_t)c.ph * p->w + c.pw) * p->c * es;
          ++n;
        }
        if (n == 4 || (i == pl.n_classes && n > 0)) {
          st = conv_halo_run_group(group, n, output, fils, firsts, stream_v);
          if (st != RB_SUCCESS) return st;
          n = 0;
        }
      }
      return RB_SUCCESS;
    }
    for (int i = 0; i < pl.n_classes; ++i) {
      const ConvPlan::StrideClass& c = pl.cls[i];
      const int k = c.ph * p->stride_w + c.pw;
      if (c.out_off == SIZE_MAX) continue;
      tb.off[k] = (long long)(c.out_off / es);
      tb.hs[k] = c.q.h; tb.wsz[k] = c.q.w;
      if (pl.cls_fused && c.pointwise) {
        st = rbGemm(&c.gemm, nullptr, output, ws + c.fil_off, ws + c.out_off, c.gemm_ws ? ws + pl.cls_ws_off : nullptr,
                    c.gemm_ws, stream_v);
        if (st != RB_SUCCESS) return st;
        continue;
      }
      if (pl.cls_fused) {
        // the unit-stride implicit GEMM of the class: "image" = output gradient, "output pixels" = the class's pixels
        ConvAOperand cv;
        cv.tensor = output;
        cv.N = p->n; cv.H = (int)ho; cv.W = (int)wo; cv.C = p->k;
        cv.P = c.q.h; cv.Q = c.q.w; cv.Y = c.q.y; cv.X = c.q.x;
        cv.stride_h = cv.stride_w = cv.dil_h = cv.dil_w = 1;
        cv.pad_h = (c.q.y - 1) - c.q.pad_h; cv.pad_w = (c.q.x - 1) - c.q.pad_w;
        cv.pad_h_hi = c.q.h - (int)ho - cv.pad_h + (c.q.y - 1);
        cv.pad_w_hi = c.q.w - (int)wo - cv.pad_w + (c.q.x - 1);
        st = gemm_run(&c.gemm, nullptr, nullptr, ws + c.fil_off, ws + c.out_off, c.gemm_ws ? ws + pl.cls_ws_off : nullptr,
                      c.gemm_ws, stream_v, &cv);
        if (st != RB_SUCCESS) return st;
        continue;
      }
      // sub-filter [g][k][j][i][c] = fil[g][k][c][y0 + stride_h * j][x0 + stride_w * i]
      const long long ssz[5] = {p->g, p->k, p->c, c.q.y, c.q.x};
      const long long sst[5] = {pl.fs[0], pl.fs[1], pl.fs[2], pl.fs[3] * p->stride_h, pl.fs[4] * p->stride_w};
      const uint8_t* first = static_cast<const uint8_t*>(filter) + (c.y0 * pl.fs[3] + c.x0 * pl.fs[4]) * (long long)es;
      permute(first, ws + c.fil_off, ssz, sst, fil_kyxc, true, es);
      st = conv_run(&c.q, -1, ws + c.fil_off, ws + c.out_off, output, ws + pl.cls_ws_off, c.ws_bytes, stream_v);
      if (st != RB_SUCCESS) return st;
    }
    // one thread per item of an image row when a row has at most 1024 items (vectors of 16 bytes where the kernel
    // can use them: the same test as inside it)
    const bool ivec = tb.s_c == 1 && (tb.C * (long long)es) % 16 == 0 && (tb.s_n * (long long)es) % 16 == 0 &&
                      (tb.s_h * (long long)es) % 16 == 0 && (tb.s_w * (long long)es) % 16 == 0 && (tb.s_g * (long long)es) % 16 == 0;
    const long long row_items = (long long)p->w * p->g * (p->c / (ivec ? (int)(16 / es) : 1));
    const int ithreads = row_items <= 1024 ? (int)((row_items + 31) / 32 * 32) : 256;
    const int ib = (int)std::min<long long>((long long)p->n * p->h, (long long)dev->sm_count * (2048 / ithreads) * 2);
    if (es == 2)
      interleave_classes_kernel<2><<<ib, ithreads, 0, stream>>>(ws, static_cast<uint8_t*>(input), tb);
    else
      interleave_classes_kernel<4><<<ib, ithreads, 0, stream>>>(ws, static_cast<uint8_t*>(input), tb);
    count_launch();
    RB_CUDA_TRY(cudaGetLastError());
    return RB_SUCCESS;
  }

  HaloConv uhc;
  const bool on_halo = !capture && unit_halo(p, pl, epi != nullptr, &uhc);
  // f32 forward on the streamed-filter halo kernel (csrc/conv_halo_stream_sm100.cu): decided here because a plain KCYX
  // filter then goes to its two K-major TF32 planes in ONE transposing pass instead of a permutation and a split.
  HaloConv f32_sc;
  long long f32_o_k = 1;
  const size_t fil_plane = up256((size_t)p->k * p->y * p->x * p->c * 4);
  const bool f32_stream = !on_halo && !capture && !epi && f32_streamed(p, pl, &f32_sc, &f32_o_k);
  const bool fil_kcyx = filter_is_kcyx(p, pl);
  const void* A;
  const void* B;
  void* C;
  const void* a_hi = input;
  const void* a_lo = nullptr;
  if (p->direction == 0 && pl.a_implicit && pl.a_planes > 0) {
    float* hi = reinterpret_cast<float*>(ws + pl.a_off);
    float* lo = pl.a_planes == 2 ? reinterpret_cast<float*>(ws + pl.a_off + pl.a_bytes / 2) : nullptr;
    const long long pix = (long long)p->n * p->h * p->w;
    if (pl.a_nchw)   // per image: [C][H*W] -> [H*W][C]
      st = f32_planes(static_cast<const float*>(input), hi, lo, p->n, p->c, p->h * p->w, p->c, true, lo != nullptr, stream_v);
    else
      st = f32_planes(static_cast<const float*>(input), hi, lo, 1, (int)pix, p->c, p->c, false, lo != nullptr, stream_v);
    if (st != RB_SUCCESS) return st;
    a_hi = hi;
    a_lo = lo;
  }
  if (p->direction == 0) {
    if (pl.a_direct) A = input; else { gather(input, ws + pl.a_off, false, false, ho, wo, p->c); A = ws + pl.a_off; }
    if (pl.b_direct) B = filter;
    else if (f32_stream && fil_kcyx) B = nullptr;   // transposed and split in one pass below
    else { permute(filter, ws + pl.b_off, fsz, pl.fs, fil_kyxc, true, es); B = ws + pl.b_off; }
    C = (pl.c_direct || pl.c_remap) ? output : static_cast<void*>(ws + pl.c_off);
  } else if (p->direction == 2) {
    if (pl.a_direct) A = output; else { permute(output, ws + pl.a_off, osz, pl.os, act_gmat, true, es); A = ws + pl.a_off; }
    if (pl.b_direct) B = input; else { gather(input, ws + pl.b_off, false, false, ho, wo, p->c); B = ws + pl.b_off; }
    C = pl.c_direct ? filter : static_cast<void*>(ws + pl.c_off);
    if (pl.w_halo && !capture && !((rbGetGemmVariant() >> 26) & 1))
      return conv_wgrad_halo_run(pl.w_hc, input, output, filter, ws + pl.gemm_off, pl.gemm_ws, stream_v);
    if (pl.b_implicit) {
      ConvAOperand cv;
      cv.operand = 1;
      cv.tensor = input;
      cv.N = p->n; cv.H = p->h; cv.W = p->w; cv.C = p->c;
      cv.P = (int)ho; cv.Q = (int)wo; cv.Y = p->y; cv.X = p->x;
      cv.stride_h = p->stride_h; cv.stride_w = p->stride_w; cv.dil_h = p->dil_h; cv.dil_w = p->dil_w;
      cv.pad_h = p->pad_h; cv.pad_w = p->pad_w; cv.pad_h_hi = p->pad_h_r; cv.pad_w_hi = p->pad_w_r;
      st = gemm_run(&pl.gemm, nullptr, A, nullptr, C, pl.gemm_ws ? ws + pl.gemm_off : nullptr, pl.gemm_ws, stream_v, &cv, capture);
      if (st != RB_SUCCESS) return st;
      if (!pl.c_direct) permute(C, filter, fsz, pl.fs, fil_kyxc, false, es_c);
      return RB_SUCCESS;
    }
  } else {
    if (pl.a_direct) A = output; else { gather(output, ws + pl.a_off, true, true, p->h, p->w, p->k); A = ws + pl.a_off; }
    if (on_halo && uhc.b_mn) {
      B = filter;   // the halo kernel takes the mirrored taps from the filter tensor itself
    } else if (pl.a_implicit) {
      // B[c][(y',x',k)] = fil[k][c][Y-1-y'][X-1-x']: walk y and x backwards from the last tap
      long long mfs[5] = {pl.fs[0], pl.fs[1], pl.fs[2], -pl.fs[3], -pl.fs[4]};
      const int fil_cyxk[5] = {0, 2, 3, 4, 1};
      const uint8_t* last_tap = static_cast<const uint8_t*>(filter) + ((p->y - 1) * pl.fs[3] + (p->x - 1) * pl.fs[4]) * (long long)es;
      permute(last_tap, ws + pl.b_off, fsz, mfs, fil_cyxk, true, es);
      B = ws + pl.b_off;
    } else if (pl.b_direct) B = filter; else { permute(filter, ws + pl.b_off, fsz, pl.fs, fil_yxkc, true, es); B = ws + pl.b_off; }
    C = pl.c_direct ? input : static_cast<void*>(ws + pl.c_off);
  }
  if (on_halo)
    return conv_halo_run(uhc, p->direction == 0 ? input : output, B, p->direction == 0 ? output : input, stream_v, epi, pl.gemm.c_type);
  // Filters too large to stay in shared memory, and f32 tensors (three TF32 products from two planes of window and
  // filter): the halo kernel with a streamed filter (csrc/conv_halo_stream_sm100.cu).
  if (!capture && !epi && pl.a_implicit && !pl.a_up && p->direction <= 1 && p->stride_h == 1 && p->stride_w == 1 &&
      !((rbGetGemmVariant() >> 26) & 1)) {
    HaloConv sc;
    halo_geometry(p, &sc);
    // (16-bit: up to 128 output channels; at 256 the GEMM kernel's 256-column MMAs run at the math rate and win:
    //  C = K = 256, 14 x 14, 3 x 3 measured 782 streamed against 970 TFLOP/s)
    if ((p->data_type == RB_F16 || p->data_type == RB_BF16) && pl.a_planes == 0 && pl.c_direct && pl.gemm.c_type == p->data_type &&
        sc.Kout <= 128 && conv_halo_stream_applicable(sc, 2, 1))
      return conv_halo_stream_run(sc, 2, p->direction == 0 ? input : output, nullptr, B, nullptr, p->direction == 0 ? output : input, 1,
                                  stream_v);
  }
  if (f32_stream) {
    float* fhi = reinterpret_cast<float*>(ws + pl.gemm_off);
    float* flo = reinterpret_cast<float*>(ws + pl.gemm_off + fil_plane);
    const int yxc = p->y * p->x * p->c;
    if (B) st = f32_planes(static_cast<const float*>(B), fhi, flo, 1, p->k, yxc, yxc, false, true, stream_v);
    else st = f32_planes(static_cast<const float*>(filter), fhi, flo, p->k, p->c, p->y * p->x, p->c, true, true, stream_v);   // per k: [C][Y*X] -> [Y*X][C]
    if (st != RB_SUCCESS) return st;
    return conv_halo_stream_run(f32_sc, 4, a_hi, a_lo, fhi, flo, output, f32_o_k, stream_v);
  }
  if (pl.a_implicit) {
    ConvAOperand cv;
    if (p->direction == 0) {
      cv.tensor = a_hi;
      cv.tensor_lo = a_lo;
      cv.N = p->n; cv.H = p->h; cv.W = p->w; cv.C = p->c;
      cv.P = (int)ho; cv.Q = (int)wo; cv.Y = p->y; cv.X = p->x;
      cv.stride_h = p->stride_h; cv.stride_w = p->stride_w; cv.dil_h = p->dil_h; cv.dil_w = p->dil_w;
      cv.pad_h = p->pad_h; cv.pad_w = p->pad_w; cv.pad_h_hi = p->pad_h_r; cv.pad_w_hi = p->pad_w_r;
      if (pl.c_remap) { cv.c_rows_per_img = (int)(ho * wo); cv.c_img_stride = pl.os[0]; cv.c_col_stride = pl.os[2]; }
    } else {
      // backward data, unit stride: "image" = output gradient (ho x wo x k), "output pixels" = input pixels (h x w)
      const int uh = ((int)ho - 1) * p->stride_h + 1, uw = ((int)wo - 1) * p->stride_w + 1;   // = ho, wo at unit stride
      cv.tensor = output;
      if (pl.a_up) {
        const int chv = (int)((size_t)p->k * es / 16);
        upsample_nhwc_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(output), reinterpret_cast<uint4*>(ws + pl.a_off),
                                                          p->n, (int)ho, (int)wo, uh, uw, chv, p->stride_h, p->stride_w);
        count_launch();
        cv.tensor = ws + pl.a_off;
      }
      cv.N = p->n; cv.H = uh; cv.W = uw; cv.C = p->k;
      cv.P = p->h; cv.Q = p->w; cv.Y = p->y; cv.X = p->x;
      cv.stride_h = 1; cv.stride_w = 1; cv.dil_h = p->dil_h; cv.dil_w = p->dil_w;
      cv.pad_h = (p->y - 1) * p->dil_h - p->pad_h; cv.pad_w = (p->x - 1) * p->dil_w - p->pad_w;
      // upper padding such that the base pixel takes exactly h (w) positions: h = ho + pad + pad_hi - (Y-1)*dil
      cv.pad_h_hi = p->h - uh - cv.pad_h + (p->y - 1) * p->dil_h;
      cv.pad_w_hi = p->w - uw - cv.pad_w + (p->x - 1) * p->dil_w;
    }
    st = gemm_run(&pl.gemm, epi, nullptr, B, C, pl.gemm_ws ? ws + pl.gemm_off : nullptr, pl.gemm_ws, stream_v, &cv, capture);
  } else {
    st = gemm_run(&pl.gemm, epi, A, B, C, pl.gemm_ws ? ws + pl.gemm_off : nullptr, pl.gemm_ws, stream_v, nullptr, capture);
  }
  if (st != RB_SUCCESS) return st;
  if (!pl.c_direct && !pl.c_remap) {
    if (p->direction == 0) permute(C, output, osz, pl.os, act_gmat, false, es_c);
    else if (p->direction == 2) permute(C, filter, fsz, pl.fs, fil_kyxc, false, es_c);
    else permute(C, input, isz, pl.is, act_gmat, false, es_c);
  }
  return RB_SUCCESS;
}
