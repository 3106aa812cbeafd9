/* The string-configured handle API of rocMLIR's kernel library (mlir/tools/rocmlir-lib/Miir.h:18-101), served
 * by the B200 kernels of rocmlir_b200. Names, argument meanings, return values and the two-call buffer protocol
 * are those of the reference; what differs is stated per function.
 *
 * Options grammar (mlir/lib/Dialect/Rock/Generator/ConvGenerator.cpp:82-98,487-668): whitespace-separated
 * `--key value` pairs. Convolutions (`--operation conv | conv_bwd_data | conv_bwd_weight`) take the reference's keys:
 *   required  arch in_type fil_type out_type in_layout fil_layout out_layout batchsize groupsize in_channels
 *             out_channels in_h in_w out_h out_w fil_h fil_w
 *   optional  dilation_h dilation_w conv_stride_h conv_stride_w padding_h padding_w kernel_id kernel_name num_cu
 *             perf_config x2 reverse_grid
 * Types: fp32 fp16 bf16 i8 (with `--out_type i32`); `fp8` (GEMM only) ; `bf8` has no kernel here: NULL handle. Layout letters in any case, `0 1` or `H W` /
 * `Y X` for the image dimensions, `N` for the filter's output-channel dimension as in the reference (GNCHW).
 * `arch` must name this hardware: `sm_100a` (also accepted: `sm_100`, `nvptx64-nvidia-cuda:sm_100a`); every other
 * architecture name, AMD ones included, gives a NULL handle, which is how the reference answers an unknown chip.
 * Extension (not in the reference's Miir): `--operation gemm` and `--operation attention` with rocmlir-gen's flag
 * names (mlir/tools/rocmlir-gen/rocmlir-gen.cpp:73-785): `t out_datatype g m n k transA transB transC`, and
 * `t g seq_len_q seq_len_k head_dim_qk head_dim_v transQ transK transV transO with-attn-scale causal`.
 *
 * Differences from the reference, by design:
 *  - a handle describes the whole operation: miirGetKernelCount() is 1 and `--kernel_id` may only be 0 (the
 *    reference needs up to 3 kernels and one handle per kernel id; the gather / reduction passes of this library
 *    are launched inside miirLaunch);
 *  - the binary of miirBufferGet is an sm_100a cubin (an ELF image for cuModuleLoadData) where the reference's is an
 *    hsaco; it holds every instantiation of the GEMM / implicit-GEMM kernel, the one a given handle launches is named
 *    by miirGetKernelLaunch, which also carries what the reference's two execution dimensions cannot: cluster size,
 *    dynamic shared memory and the parameter block with the TMA tensor maps of the caller's buffers;
 *  - operations that run as several kernels (layout, filter or reduction passes beside the GEMM kernel; attention)
 *    are launched through miirLaunch, or later through miirLaunchFromBuffer from the small relocatable descriptor of
 *    miirDescriptorGet (problem + tile configuration), in place of the client's own hipModuleLaunchKernel.
 */
#ifndef MIIR_B200_H
#define MIIR_B200_H

#include <stddef.h>
#include <stdint.h>

#include "rocmlir_b200.h" /* RbKernelLaunch */

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MIIR_EXPORT __attribute__((visibility("default")))
#else
#define MIIR_EXPORT
#endif

/* Miir.h:16: version 6 = kernels take bare pointers. Kept. */
#define MIIR_VERSION_FLAT 6

/* Miir.h:20-26 */
enum MiirStatus { MIIR_SUCCESS = 0, MIIR_INVALID_PARAM, MIIR_INVALID_MODULE, MIIR_BUILD_FAILURE };
typedef enum MiirStatus MiirStatus;

/* Miir.h:30 */
typedef void *MiirHandle;

/* Miir.h:50: NULL when the options are incomplete, inconsistent (dimension check of
 * ConvGenerator.cpp:139-245), or name something this library has no kernel for. */
MIIR_EXPORT MiirHandle miirCreateHandle(const char *options);

/* Miir.h:56: -1 for a NULL handle. Always 1 here (see above). */
MIIR_EXPORT int miirGetKernelCount(MiirHandle handle);

/* Miir.h:65: bytes of device workspace the operation needs; 0 for a NULL handle. */
MIIR_EXPORT int miirGetWorkspaceSize(MiirHandle handle);

/* Miir.h:70: selects the tile configuration (the applicability + tuning-parameter part of lowering). */
MIIR_EXPORT MiirStatus miirLowerTuningParams(MiirHandle handle);

/* Miir.h:75: the same selection; afterwards miirBufferGet / miirGetKernelLaunch / miirDescriptorGet answer. */
MIIR_EXPORT MiirStatus miirLowerBin(MiirHandle handle);

/* Miir.h:89: two-call protocol. buffer == NULL: *size receives the size of the code object; otherwise the code
 * object - the library's sm_100a cubin - is copied into buffer. MIIR_INVALID_PARAM when both are NULL or the handle is
 * NULL; MIIR_INVALID_MODULE before miirLowerBin; MIIR_BUILD_FAILURE for an attention handle (its kernels are launched
 * through miirLaunch only). */
MIIR_EXPORT MiirStatus miirBufferGet(MiirHandle handle, char *buffer, size_t *size);

/* What the reference's {code object, global size, local size} cannot say on this hardware (no counterpart in Miir.h):
 * for the buffers arg0..arg2 (kernel-argument order: filter, input, output / a, b, c) the name of the handle's
 * kernel inside the cubin, its cluster size, dynamic shared memory and parameter block. See RbKernelLaunch in
 * rocmlir_b200.h for how to launch it with cuLaunchKernelEx. MIIR_BUILD_FAILURE when the operation does not run as
 * one kernel (then use miirLaunch); MIIR_INVALID_MODULE before miirLowerBin. Needs the GPU (tensor maps are
 * encoded by the driver). */
MIIR_EXPORT MiirStatus miirGetKernelLaunch(MiirHandle handle, void *arg0, void *arg1, void *arg2, RbKernelLaunch *out);

/* The relocatable launch descriptor of the whole operation (problem + tile configuration, a few hundred bytes), same
 * two-call protocol: what a client's kernel cache keeps for miirLaunchFromBuffer. No counterpart in Miir.h. */
MIIR_EXPORT MiirStatus miirDescriptorGet(MiirHandle handle, char *buffer, size_t *size);

/* Miir.h:97: global_size = grid * block and local_size = block of the operation's GEMM kernel (1-D).
 * MIIR_INVALID_MODULE before one of the miirLower* calls. */
MIIR_EXPORT MiirStatus miirGetExecutionDims(MiirHandle handle, size_t *global_size, size_t *local_size);

/* Miir.h:101 */
MIIR_EXPORT MiirStatus miirDestroyHandle(MiirHandle handle);

/* Bytes of the operation's tensors in argument order (convolution: filter, input, output; GEMM: A, B, C; attention:
 * Q, K, V and, in sizes[3], O), sizes = size_t[4]. No reference counterpart: the reference's tuning driver reads them
 * off the kernel's signature (mlir/tools/rocmlir-tuning-driver/rocmlir-tuning-driver.cpp:131-185). */
MIIR_EXPORT MiirStatus miirGetArgSizes(MiirHandle handle, size_t *sizes);

/* ---- launch (no reference counterpart: the reference's clients load the code object and launch it themselves) ----
 * Arguments in the kernel-argument order of the reference (ConvGenerator.cpp:788-1024): filter, input, output for
 * all three convolution directions; a, b, c for gemm; for attention q, k, v in the first three slots and o in
 * `extra`. `workspace` must hold miirGetWorkspaceSize() bytes. Returns MIIR_INVALID_MODULE before a miirLower*
 * call, MIIR_BUILD_FAILURE when the launch fails (text: rbGetLastError of rocmlir_b200.h). */
MIIR_EXPORT MiirStatus miirLaunch(MiirHandle handle, void *arg0, void *arg1, void *arg2, void *extra, void *workspace,
                                  size_t workspace_bytes, void *stream);

/* The same from a descriptor obtained with miirDescriptorGet (e.g. out of a client's kernel cache). */
MIIR_EXPORT MiirStatus miirLaunchFromBuffer(const char *buffer, size_t size, void *arg0, void *arg1, void *arg2,
                                            void *extra, void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MIIR_B200_H */
