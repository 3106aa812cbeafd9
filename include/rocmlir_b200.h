/* rocmlir_b200 — C ABI of the B200 (sm_100a) contraction-kernel library.
 *
 * The library stands behind the boundary that rocMLIR offers to MIGraphX / MIOpen-style clients:
 * where the reference lowers one fused kernel function to an AMD code object and hands back
 * {binary, block size, grid size}, this library selects a hand-written sm_100a kernel and either
 * launches it (rb* entry points below) or describes it (miir* entry points, Miir-compatible).
 *
 * Plain C: pointers and sizes only. Device pointers are ordinary CUDA device addresses; `stream`
 * is a cudaStream_t passed as void* (NULL = default stream). Nothing here allocates device memory
 * on the caller's behalf except where a function says so.
 */
#ifndef ROCMLIR_B200_H
#define ROCMLIR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RB_API_VERSION 2

#if defined(__GNUC__)
#define RB_EXPORT __attribute__((visibility("default")))
#else
#define RB_EXPORT
#endif

/* Element types. Mirrors the type names rocmlir-gen accepts for -t / -out_datatype
 * (mlir/tools/rocmlir-gen/rocmlir-gen.cpp:432-458): f32 f16 bf16 i8 i32 fp8 (OCP e4m3fn). */
typedef enum RbDType {
  RB_F32 = 0,
  RB_F16 = 1,
  RB_BF16 = 2,
  RB_I8 = 3,
  RB_I32 = 4,
  RB_F8E4M3 = 5,
  /* GEMM inputs only (results are f32 / f16 / bf16): OCP e5m2 ("bf8"), and the two mixed pairs rocmlir-gen spells
   * fp8_bf8 (A e4m3, B e5m2) and bf8_fp8 (A e5m2, B e4m3). */
  RB_F8E5M2 = 6,
  RB_F8E4M3_E5M2 = 7,
  RB_F8E5M2_E4M3 = 8
} RbDType;

typedef enum RbStatus {
  RB_SUCCESS = 0,
  RB_INVALID_PARAM = 1,   /* malformed problem (sizes <= 0, unknown dtype, NULL pointer) */
  RB_UNSUPPORTED = 2,     /* well-formed, but no kernel for it: the "applicability" failure of
                             mlirMIGraphXAddApplicabilityPipeline (mlir-c/Dialect/MIGraphX.h:66-73) */
  RB_WORKSPACE_TOO_SMALL = 3,
  RB_CUDA_ERROR = 4,
  RB_KERNEL_TIMEOUT = 5   /* a bounded device-side wait ran out. Returned by the synchronous entry points (rbGemmHost);
                             the asynchronous ones return before the kernel ends: poll rbReadKernelStatus */
} RbStatus;

/* Fused elementwise epilogue applied to the accumulator tile before the single global store.
 * Replaces the linalg.generic readers that rocMLIR re-tiles onto the accumulator registers
 * (mlir/lib/Dialect/Rock/Transforms/AlignTiling.cpp:903-1049) for the forms MIGraphX emits:
 * dequantizelinear / quantizelinear / add(broadcast bias) / relu / convert
 * (mlir/lib/Conversion/MIGraphXToTosa/MIGraphXToTosa.cpp:876-1018).
 *
 * Order of evaluation, each step an individually rounded f32 (or `mid_type`) operation:
 *   x = acc                       (f32, or i32 -> f32 round-to-nearest-even when any float step is on)
 *   x = x - in_zero               if RB_EPI_ZP_IN      (dequantizelinear zero point, cast to f32 by the caller:
 *                                                       (cast(x) - cast(zp)) * scale, MIGraphXToTosa.cpp:879-902)
 *   x = round_to(mid_type, x)     if RB_EPI_ROUND_MID  (the GEMM's declared result type)
 *   x = x * alpha                 if RB_EPI_ALPHA      (per-tensor scale product, fp8)
 *   x = x * col_scale[n]          if RB_EPI_COL_SCALE  (per-column dequantisation scale, f32)
 *   x = x + bias[n]               if RB_EPI_BIAS       (then round_to(mid_type) if ROUND_MID); with RB_EPI_BIAS_ROW the
 *                                                       vector is indexed by the row m (a bias broadcast along N), with
 *                                                       RB_EPI_BIAS_SCALAR it is the single element bias[0]
 *   x = x + residual[g][m][n]     if RB_EPI_RESIDUAL   (a tensor of C's shape and layout: the same-shape add of
 *                                                       mixr-gemm-add; then round_to(mid_type) if ROUND_MID)
 *   x = f(x)                      if RB_EPI_UNARY      (one of the MIGraphX unary elementwise ops, `unary` = RbUnary:
 *                                                       mlir/include/mlir/Dialect/MIGraphX/IR/MIGraphX.td:134-181; evaluated in f32,
 *                                                       then round_to(mid_type) if ROUND_MID)
 *   x = max(x, 0)                 if RB_EPI_RELU
 *   x = min(max(x, lo), hi)       if RB_EPI_CLIP       (migraphx.clip, MIGraphXToTosa.cpp:1089-1101)
 *   x = x * out_recip             if RB_EPI_REQUANT    (out_recip = 1/scale computed by the caller in f32)
 *   store: convert x to the C type (floats: RNE, fp8 saturating; integers: RNE then saturate; i8 with
 *          RB_EPI_ZP_OUT: cast to i32, + out_zero, clamp to [-128, 127], MIGraphXToTosa.cpp:908-982). */
enum {
  RB_EPI_ALPHA = 1,
  RB_EPI_COL_SCALE = 2,
  RB_EPI_BIAS = 4,
  RB_EPI_RELU = 8,
  RB_EPI_REQUANT = 16,
  RB_EPI_ROUND_MID = 32,
  RB_EPI_CLIP = 64,
  RB_EPI_RESIDUAL = 128,
  RB_EPI_BIAS_ROW = 256,
  RB_EPI_BIAS_SCALAR = 512,
  RB_EPI_ZP_IN = 1024,
  RB_EPI_ZP_OUT = 2048,
  RB_EPI_UNARY = 4096
};

/* RbEpilogue::unary (migraphx.abs / ceil / erf / exp / floor / log / neg / recip / rsqrt / sigmoid / sqrt / tanh) */
typedef enum RbUnary {
  RB_UNARY_NONE = 0, RB_UNARY_ABS, RB_UNARY_CEIL, RB_UNARY_ERF, RB_UNARY_EXP, RB_UNARY_FLOOR, RB_UNARY_LOG, RB_UNARY_NEG,
  RB_UNARY_RECIP, RB_UNARY_RSQRT, RB_UNARY_SIGMOID, RB_UNARY_SQRT, RB_UNARY_TANH
} RbUnary;

typedef struct RbEpilogue {
  uint32_t flags;
  float alpha;
  float out_recip;
  int32_t mid_type;        /* RbDType used by RB_EPI_ROUND_MID */
  int32_t bias_type;       /* RbDType of bias[]: RB_F32, RB_F16 or RB_BF16 */
  const float *col_scale;  /* device, [n] */
  const void *bias;        /* device, [n] ([m] with RB_EPI_BIAS_ROW, one element with RB_EPI_BIAS_SCALAR) */
  float clip_lo, clip_hi;  /* RB_EPI_CLIP */
  float in_zero;           /* RB_EPI_ZP_IN */
  int32_t out_zero;        /* RB_EPI_ZP_OUT */
  const void *residual;    /* device, C's shape and layout (also under trans_c) */
  int32_t res_type;        /* RbDType of residual[]: RB_F32, RB_F16 or RB_BF16 */
  int32_t unary;           /* RbUnary, RB_EPI_UNARY (occupies what was tail padding: the struct's size is unchanged) */
} RbEpilogue;

/* rock.gemm (mlir/include/mlir/Dialect/Rock/IR/RockOps.td:136-181):
 *   C[g,m,n] = sum_k A[g,m,k] * B[g,k,n]
 * A is stored G x M x K (trans_a: G x K x M), B is G x K x N (trans_b: G x N x K), C is G x M x N
 * (trans_c: G x N x M); every matrix row-major and contiguous, exactly the flat buffers that
 * rocmlir-gen's kernels take (rocmlir-gen.cpp:2094-2124). Accumulation is f32 for float inputs
 * and i32 for i8 (mlir/lib/Dialect/Rock/Transforms/GemmToGridwise.cpp:93-109). */
typedef struct RbGemmProblem {
  int32_t g, m, n, k;
  int32_t trans_a, trans_b, trans_c;
  int32_t ab_type; /* RbDType of A and B */
  int32_t c_type;  /* RbDType of C */
  int32_t f32_mode; /* for ab_type RB_F32: 0 = 3xTF32 split (fp32-class accuracy), 1 = single TF32 pass */
  int32_t store_method; /* 0 = set: C = A.B; 1 = add: C = C + A.B on a C the caller has filled (rock.gemm's
                           store_method = atomic_add, rocmlir-gen --store-method, rocmlir-gen.cpp:325-331). The product is
                           rounded to C's type and added in it; f32 / f16 / bf16 results. Deterministic: no atomics. */
} RbGemmProblem;

/* Bytes of caller-provided device workspace rbGemm needs for this problem (0 for most). */
RB_EXPORT size_t rbGemmWorkspaceSize(const RbGemmProblem *p);

/* Runs the GEMM on `stream`. Returns RB_UNSUPPORTED for problems outside the kernel's reach. */
RB_EXPORT RbStatus rbGemm(const RbGemmProblem *p, const RbEpilogue *epi /* may be NULL */, const void *a, const void *b,
                void *c, void *workspace, size_t workspace_bytes, void *stream);

/* rbGemm for callers that cannot allocate device memory. (No counterpart in the reference: there the client
 * owns every buffer, workspace included.)
 *
 * Some hosts of this library are not allowed to call cudaMalloc at the point where they need a GEMM: code that
 * runs inside a memory-pool or allocator callback, a plugin that is handed its buffers by a framework and must
 * not grow the process's device footprint, a real-time loop that may not take the allocator's lock. rbGemm asks
 * such callers for a workspace whenever it pads an operand whose row pitch is not a multiple of 16 bytes,
 * splits f32 operands into TF32 planes, or cuts K into ranges; this entry point takes no workspace and uses a
 * fixed RB_NO_ALLOC_SCRATCH_BYTES array inside the library image instead. It calls no cudaMalloc, cudaFree or
 * allocating library routine. The inputs and the output are still the caller's.
 *
 *  - Problems whose scratch need (rbGemmWorkspaceSize) exceeds RB_NO_ALLOC_SCRATCH_BYTES are rejected with
 *    RB_WORKSPACE_TOO_SMALL and a message naming both sizes; nothing is launched.
 *  - The first call on each device looks up the scratch array's device address (cudaGetSymbolAddress, with that
 *    device current). Make that first call before any stream capture begins.
 *  - All calls on a device share the one array and it keeps the previous call's contents. The kernels overwrite
 *    every byte they later read, so nothing has to be cleared; but two calls whose kernels overlap on the GPU
 *    (different streams, or different host threads) race on it. Serialise such calls on one stream.
 *  - Every GPU that loads the library holds the array until the process exits. */
#define RB_NO_ALLOC_SCRATCH_BYTES (16u << 20)
RB_EXPORT RbStatus rbGemmNoAlloc(const RbGemmProblem *p, const RbEpilogue *epi /* may be NULL */, const void *a,
                                 const void *b, void *c, void *stream);

/* Same operation on HOST buffers: copies A and B (and the epilogue vectors, whose pointers are host
 * pointers here) to the device, runs rbGemm, copies C back and waits for `stream`. Counterpart of the
 * `<kernel>_gpu` wrapper of rocmlir-gen's host harness (mlir/tools/rocmlir-gen/rocmlir-gen.cpp:1211-1283).
 * Device staging memory is a grow-only arena owned by the calling thread (cudaMalloc on first use or growth). */
RB_EXPORT RbStatus rbGemmHost(const RbGemmProblem *p, const RbEpilogue *epi_host /* may be NULL */, const void *a_host,
                              const void *b_host, void *c_host, void *stream);

/* rock.conv / rock.conv_bwd_data / rock.conv_bwd_weight
 * (mlir/include/mlir/Dialect/Rock/IR/RockOps.td:87-134). Tensors are 5-D with an explicit group dimension,
 * each stored in the order its layout string spells, as ConvGenerator canonicalises them
 * (mlir/lib/Dialect/Rock/Generator/ConvGenerator.cpp:487-668): filter letters g k c y x, input n g c h w,
 * output n g k h w (e.g. "gkyxc" / "nhwgc" / "nhwgk" for NHWC, "gkcyx" / "ngchw" / "ngkhw" for NCHW).
 * c and k count channels PER GROUP. in_h = ho * stride_h + y * dil_h - pad_h, and ho, wo must equal
 * (in + pad + pad_r - (fil - 1) * dil - 1) / stride + 1 (ConvGenerator.h:98-104).
 * Argument order is (filter, input, output) for all three directions, as in the reference's kernels
 * (ConvGenerator.cpp:825-830); the direction decides which one is written:
 *   0 forward: output; 1 backward data: input; 2 backward weight: filter.
 * i8 (forward only) produces an i32 output and the 8-bit floats RB_F8E4M3 / RB_F8E5M2 (forward only) an f32
 * output, like rocmlir-gen's -t i8 / fp8 / bf8 (rocmlir-gen.cpp:430-455). */
typedef struct RbConvProblem {
  int32_t n, g, c, k;
  int32_t h, w, y, x;
  int32_t stride_h, stride_w, dil_h, dil_w;
  int32_t pad_h, pad_w, pad_h_r, pad_w_r;
  int32_t ho, wo;
  int32_t data_type; /* RbDType of filter, input and output (i8: output is i32) */
  int32_t direction;
  int32_t f32_mode;  /* as in RbGemmProblem */
  char fil_layout[8], in_layout[8], out_layout[8];
} RbConvProblem;

/* Bytes of device workspace rbConv needs (gathered operand matrices, split-K planes); the counterpart of
 * miirGetWorkspaceSize (mlir/tools/rocmlir-lib/Miir.h:60-66). 0 also for an invalid problem. */
RB_EXPORT size_t rbConvWorkspaceSize(const RbConvProblem *p);

/* Number of kernels one rbConv call launches besides those inside its GEMM (counterpart of
 * miirGetKernelCount, Miir.h:54-58); -1 for an invalid problem. */
RB_EXPORT int rbConvKernelCount(const RbConvProblem *p);

/* The GEMM a convolution is computed as (the reference's GemmSize::fromConvolution and the backward variants,
 * mlir/lib/Dialect/Rock/IR/RockDialect.cpp:509-533,671-749): forward M = N*Ho*Wo, N = K, K = Y*X*C; backward
 * data M = N*H*W, N = C, K = Y*X*K; backward weight M = K, N = Y*X*C, K = N*Ho*Wo (per group). */
RB_EXPORT RbStatus rbConvGetGemmProblem(const RbConvProblem *p, RbGemmProblem *out);

RB_EXPORT RbStatus rbConv(const RbConvProblem *p, void *filter, void *input, void *output, void *workspace,
                          size_t workspace_bytes, void *stream);

/* Forward convolution with the fused elementwise tail MIGraphX attaches to it (convolution + broadcast add +
 * relu / clip: mlir/test/CAPI/mixr_full.c:88-159, mlir/test/fusion/pr-e2e/mixr-conv-bias-clipped-relu.mlir:5-13;
 * quant_convolution -> dequantizelinear -> ... -> quantizelinear: mlir/test/fusion/pr-e2e/tosa-to-rock-quantization.e2e.mlir).
 * The epilogue is RbEpilogue as for rbGemm, with the output channel k in the place of the column n (bias[k],
 * col_scale[k]); a residual operand has the output tensor's shape and needs the "nhwgk" output layout. `out_type` is
 * the element type of the output tensor after the epilogue (an RbDType, e.g. RB_I8 for a requantised i8 convolution),
 * -1 for the type rbConv would write. Forward direction only (the reference fuses nothing into the backward ops). */
RB_EXPORT size_t rbConvEpiWorkspaceSize(const RbConvProblem *p, int32_t out_type);
RB_EXPORT RbStatus rbConvEpi(const RbConvProblem *p, const RbEpilogue *epi /* may be NULL */, int32_t out_type, void *filter,
                             void *input, void *output, void *workspace, size_t workspace_bytes, void *stream);

/* The same three operations with a third image dimension (depth), as rocmlir-gen builds them for layouts with
 * three image letters (mlir/tools/rocmlir-gen/rocmlir-gen.cpp:3545-3581; letters and their digit aliases in
 * mlir/lib/Dialect/Rock/Generator/ConvGenerator.cpp:622-627): filter letters g k c z y x, input n g c d h w,
 * output n g k d h w, each a 6-letter permutation. Index relation and size rule per dimension are rbConv's.
 * A problem whose depths are all 1 is the 2-D problem on the same bytes and runs as such. Otherwise the depth is
 * folded: the filter depth taps become extra input channels of a 2-D convolution over N * Do images
 * (in2[g,(n,do),h,w,(z,c)] = in[n,g,c,do*stride_d + z*dil_d - pad_d,h,w], zero outside), with one gather pass
 * before and one permuting pass after the 2-D kernels; backward data sums the Z taps of every input voxel in f32. */
typedef struct RbConv3dProblem {
  int32_t n, g, c, k;
  int32_t d, h, w, z, y, x;
  int32_t stride_d, stride_h, stride_w, dil_d, dil_h, dil_w;
  int32_t pad_d, pad_h, pad_w, pad_d_r, pad_h_r, pad_w_r;
  int32_t dout, ho, wo;
  int32_t data_type; /* as in RbConvProblem */
  int32_t direction;
  int32_t f32_mode;
  char fil_layout[8], in_layout[8], out_layout[8];
} RbConv3dProblem;

RB_EXPORT size_t rbConv3dWorkspaceSize(const RbConv3dProblem *p);
RB_EXPORT RbStatus rbConv3d(const RbConv3dProblem *p, void *filter, void *input, void *output, void *workspace,
                            size_t workspace_bytes, void *stream);

/* rock.attention (mlir/include/mlir/Dialect/Rock/IR/RockOps.td:208-254): per group g
 *   O = softmax_k( f(Q . K) ) . V      Q [G][Sq][D], K [G][D][Sk] (trans_k: [G][Sk][D]), V [G][Sk][Dv], O [G][Sq][Dv]
 * the buffers of rocmlir-gen's rock_attention kernel (rocmlir-gen.cpp:2149-2200, 2264-2328). The reference has no
 * 1/sqrt(d) and no mask inside the op: callers put them into the elementwise region f between the two products
 * (TosaToRock.cpp:779-1074). Here f is:  s*scale (has_scale: the MIGraphX scalar-literal form)  * scale_tensor[g][q][k]
 * (optional)  + bias[g][q][k]
 * (optional, element type)  then  where(mask[g][q][k] != 0, s, mask_fill) (optional, i8: the mixr-attn-where form)
 * then, with `causal`, keys k > q are dropped analytically (equal to a lower-triangular mask with fill -inf, without
 * reading a [G][Sq][Sk] tensor). Row statistics are f32. f16 and bf16 (and the i8 form below) with head dimensions
 * multiples of 8 up to 128; f32 (any head dimension) runs as three kernels in true f32 - both products on the FMA
 * pipe in the reference's operation order around a row softmax - with the score matrix in scratch. trans_q / trans_v / trans_o mean Q [G][D][Sq], V [G][Dv][Sk], O [G][Dv][Sq]
 * (rocmlir-gen's -transQ / -transV / -transO); those, and a K [G][D][Sk] whose rows do not start on 16-byte
 * boundaries, cost one re-striding pass each in scratch memory the calling thread owns. */
typedef struct RbAttentionProblem {
  int32_t g, seq_q, seq_k, head_qk, head_v;
  int32_t trans_q, trans_k, trans_v, trans_o;
  int32_t data_type;
  int32_t has_scale;
  float scale;
  int32_t causal;
  float mask_fill;
  const void *bias;
  const int8_t *mask;
  const void *scale_tensor; /* optional [G][Sq][Sk] of the element type: s * scale_tensor[g][q][k] before the bias
                               (rocmlir-gen's --with-attn-scale operand, rocmlir-gen.cpp:2338-2391) */
  /* data_type RB_I8: the first-GEMM-quantised form (rocmlir-gen -t i8, rocmlir-gen.cpp:3497-3515): Q and K are
   * i8, V, O, scale_tensor and bias f16, and the scores are (i32(Q.K) - quant_bias[0]) cast to f16, times
   * quant_scale[0] (rocmlir-gen.cpp:2353-2366), before scale, bias and softmax. Both are device pointers to the
   * single element of the reference's 1x1x1 operands (i8 and f16) and are required for RB_I8, ignored otherwise.
   * Q and K are widened to f16 (exact) in scratch memory the calling thread owns (grow-only, cudaMalloc on growth). */
  const void *quant_bias;
  const void *quant_scale;
} RbAttentionProblem;

/* Scratch: operands the kernels cannot load as they lie (i8 Q / K, transposed Q / V / O, a K whose rows are off
 * 16-byte boundaries) are staged, and the f32 form keeps its G x Sq x Sk score matrix, in scratch memory.
 * rbAttentionWs takes that memory from the caller like rbGemm and rbConv do: rbAttentionWorkspaceSize bytes (0 for
 * the plain f16 / bf16 form), 16-byte aligned; it allocates nothing, so it may be captured into a CUDA graph and
 * calls on different streams may overlap when each has its own workspace.
 * rbAttention is the same call with scratch owned by the calling thread: one grow-only block per host thread, grown
 * with cudaDeviceSynchronize + cudaFree + cudaMalloc inside the call and kept until the thread exits (1 GiB for an f32
 * problem with G = 64, S = 2048). Because of that block, rbAttention calls that need scratch must not overlap on the
 * GPU when issued by one host thread (two streams would race on it) and must not be made during stream capture when
 * the block may grow; forms that need no scratch have neither restriction. */
RB_EXPORT size_t rbAttentionWorkspaceSize(const RbAttentionProblem *p);
RB_EXPORT RbStatus rbAttentionWs(const RbAttentionProblem *p, const void *q, const void *k, const void *v, void *o,
                                 void *workspace, size_t workspace_bytes, void *stream);
RB_EXPORT RbStatus rbAttention(const RbAttentionProblem *p, const void *q, const void *k, const void *v, void *o,
                               void *stream);

/* int4 operands (migraphx.unpack + dequantizelinear in front of a contraction: mlir/include/mlir/Dialect/MIGraphX/IR/
 * MIGraphX.td:183-212, mlir/lib/Dialect/MIGraphX/Transforms/RealizeInt4.cpp). `packed` holds two 4-bit values per byte
 * along the contiguous dimension; out[2i] = (low nibble - zero_point) * scale, out[2i+1] = (high nibble - zero_point) *
 * scale, rounded once to out_type (RB_F16, RB_BF16, RB_F32), or the plain sign- / zero-extended values for RB_I8
 * (scale and zero_point unused). `out` has 2 * packed_bytes elements and then is an ordinary operand of rbGemm / rbConv.
 * The reference fuses this into its operand loads; here it is one pass through memory. */
RB_EXPORT RbStatus rbUnpackInt4(const void *packed, void *out, int64_t packed_bytes, int32_t is_unsigned, int32_t out_type,
                                float scale, int32_t zero_point, void *stream);

/* GEMM + GEMM: O[g] = (A[g] . B1[g]) . B2[g], A G x M x K1, B1 G x K1 x N1, B2 G x N1 x N2, O G x M x N2, the
 * intermediate rounded to the element type, both products accumulated in f32 — the attention skeleton of the
 * reference with the softmax removed (mlir/include/mlir/Dialect/Rock/IR/Rock.h:52-56,
 * mlir/lib/Dialect/Rock/Transforms/GridwiseGemmToBlockwise.cpp:1790-1813). With k1, n2 <= 128 the intermediate stays
 * on the SM (one launch, no workspace use); otherwise it is kept in `workspace` (which must not overlap the operands),
 * written and read by one chained launch when k1 = n1 = n2 (16-bit types; the workspace then also holds the flag
 * words that order the two products) and by two launches for other extents. */
RB_EXPORT size_t rbGemmGemmWorkspaceSize(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type);
RB_EXPORT RbStatus rbGemmGemm(int32_t g, int32_t m, int32_t k1, int32_t n1, int32_t n2, int32_t data_type, const void *a,
                              const void *b1, const void *b2, void *o, void *workspace, size_t workspace_bytes,
                              void *stream);

/* ---- The kernels as a loadable binary ------------------------------------------------------------------------------
 * Where the reference hands its client a code object plus {block size, grid size} (mlirGetBinary / mlirGetKernelAttrs,
 * mlir/include/mlir-c/Dialect/MIGraphX.h:48-56; miirBufferGet, mlir/tools/rocmlir-lib/Miir.h:89) and the client
 * launches it itself, this library hands out an sm_100a cubin (an ELF image for cuModuleLoadData) that holds every
 * instantiation of its GEMM / implicit-GEMM-convolution kernel, and describes the launch of one problem in
 * RbKernelLaunch: what the two integers of the reference cannot carry on this hardware - the kernel's name inside the
 * image, the cluster size (cuLaunchKernelEx, CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION), the dynamic shared memory
 * (CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES and the launch) and the kernel's parameter block, which contains
 * the TMA tensor maps with the device addresses of the operands encoded (so it is made per set of buffers).
 * Launch: kernelParams[i] = params + param_offset[i] for i < param_count; grid (grid,1,1), block (block,1,1).
 * Only problems that run as ONE kernel have such a description (no operand copy, TF32 planes, K split, layout or
 * filter pass): the others return RB_UNSUPPORTED here and are launched through rbGemm / rbConv. */
typedef struct RbKernelLaunch {
  char symbol[160];
  uint32_t grid, block;
  uint32_t cluster;            /* CTAs per cluster along x: 1 or 2 */
  uint32_t dynamic_smem;       /* bytes */
  uint32_t param_count;        /* 2 */
  uint32_t param_offset[4], param_size[4];
  uint32_t reserved[3];
  unsigned char params[2048] __attribute__((aligned(64)));
} RbKernelLaunch;

RB_EXPORT RbStatus rbGetKernelBinary(const void **image, size_t *size);
RB_EXPORT RbStatus rbGemmEncodeLaunch(const RbGemmProblem *p, const RbEpilogue *epi /* may be NULL */, const void *a,
                                      const void *b, void *c, RbKernelLaunch *out);
RB_EXPORT RbStatus rbConvEncodeLaunch(const RbConvProblem *p, const RbEpilogue *epi /* may be NULL */, int32_t out_type,
                                      void *filter, void *input, void *output, RbKernelLaunch *out);

/* Kernel-selection knob for tuning/experiments: tile variant used by subsequent rbGemm calls on this
 * thread's library state. 0 = automatic (measured table). Mirrors the role of rocMLIR's perf_config
 * (mlir/include/mlir/Dialect/Rock/Tuning/GridwiseGemmParams.h:138-194). */
RB_EXPORT void rbSetGemmVariant(int variant);
RB_EXPORT int rbGetGemmVariant(void);

/* The tile configuration the library would launch for `p` under the calling thread's variant word (on a
 * 148-SM B200): the information rocMLIR attaches to a lowered kernel as block_size / grid_size attributes
 * (mlir/lib/Dialect/Rock/Transforms/AffixTuningParameters.cpp:69-87) plus what a 1-D launch cannot carry on
 * this hardware (dynamic shared memory, CTAs per cluster). Planned for the SM count of the current device (148
 * without one). `variant` is the explicit variant word that
 * reproduces the configuration. */
typedef struct RbGemmConfigInfo {
  int32_t tile_m, tile_n, tile_k; /* output tile of one CTA group; K elements per pipeline stage */
  int32_t ctas;                   /* CTAs per cluster (1, or 2 = cta_group::2 pair) */
  int32_t stages;                 /* depth of the shared-memory ring */
  int32_t splits;                 /* K ranges (1 = no split) */
  int32_t stream_k;               /* 1 when the stream-K tail is active */
  uint32_t grid, block;           /* 1-D launch: CTAs and threads per CTA */
  uint32_t dynamic_smem;          /* bytes, for a call without per-column epilogue vectors */
  uint32_t variant;               /* reproduces tile, CTAs, ring depth, K split, stream-K and kpr when set explicitly */
  int32_t kpr;                    /* K blocks per barrier round of the ring (1, 2 or 4) */
  int32_t stages_epi_vec;         /* ring depth and dynamic shared memory of the same problem when the epilogue */
  uint32_t dynamic_smem_epi_vec;  /* carries bias[] or col_scale[] (their staging takes room from the ring) */
} RbGemmConfigInfo;
RB_EXPORT RbStatus rbGemmGetConfig(const RbGemmProblem *p, RbGemmConfigInfo *out);

/* Tracing: when a device buffer of at least 16 * (CTAs of the launch) 64-bit words is set, the GEMM kernel
 * writes per-CTA SM-cycle counters into it: [1] producer waited for a free stage, [2] MMA thread waited for
 * loaded data, [3] MMA thread waited for a free accumulator, [4] MMA loop total, [5] tiles, [6] epilogue
 * waited for a tile, [7] epilogue busy, [8..14] cumulative [2] after each of the first 7 tiles, [15] the MMA loop in nanoseconds. NULL switches tracing off. Thread-local, like the variant knob.
 * The reference's counterpart is external profiling (rocprof) around mlir-cpu-runner
 * (mlir/utils/performance/perfRunner.py:131-150). */
RB_EXPORT void rbSetTraceBuffer(unsigned long long *device_buf, size_t n_u64);

/* Device status word: 0 when every bounded wait completed. Synchronises the device. */
RB_EXPORT RbStatus rbReadKernelStatus(uint32_t *status_out, int clear);

/* Budget of every bounded device-side wait of the GEMM kernel (mbarrier and flag waits of all roles) for launches
 * made by the calling thread, in SM clock cycles; 0 restores the default of about two seconds. When a wait runs
 * out the role records a code in the status word, the CTA frees its tensor memory and returns: the context stays
 * usable and the next launch works. The reference has no counterpart (a hung kernel there is the runtime's). */
RB_EXPORT void rbSetWaitLimit(uint64_t sm_cycles);

/* Failure-detection test hook: the next `launches` GEMM kernels launched by the calling thread issue no operand
 * loads, so that every wait of every role runs out after the wait limit and the kernel returns with a nonzero
 * status word and an undefined result. Injected on the host; nothing faults or hangs. */
RB_EXPORT void rbInjectStall(int launches);

/* Number of kernel launches this library issued since load (a monotone counter). */
RB_EXPORT uint64_t rbLaunchCount(void);

/* Last error text for this thread (never NULL). */
RB_EXPORT const char *rbGetLastError(void);

#ifdef __cplusplus
}
#endif
#endif /* ROCMLIR_B200_H */
