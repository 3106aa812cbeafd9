// Every instantiation of the tcgen05 GEMM / implicit-GEMM kernel, compiled to one sm_100a cubin (nvcc -cubin) and
// linked into the library as data: the code object that rbGetKernelBinary / miirBufferGet / mlirGetBinary hand to
// clients that load and launch kernels themselves, as rocMLIR's clients do with its hsaco
// (mlir/lib/CAPI/Dialect/MIGraphX.cpp:114-132, mlir/tools/rocmlir-lib/rocmlir-lib.cpp:292-316).
// The kernel source is the one the library launches itself (gemm_sm100.cuh), so both paths run identical code.
#include "../gemm_sm100.cuh"

namespace rb {
#define RB_INST(KIND, A, B, C) \
  template __global__ void gemm_tcgen05_kernel<KIND, A, B, C, false>(const __grid_constant__ GemmTensorMaps, const GemmParams); \
  template __global__ void gemm_tcgen05_kernel<KIND, A, B, C, true>(const __grid_constant__ GemmTensorMaps, const GemmParams);
#define RB_INST_MAJORS(KIND, C) RB_INST(KIND, false, false, C) RB_INST(KIND, false, true, C) RB_INST(KIND, true, false, C) RB_INST(KIND, true, true, C)
RB_INST_MAJORS(kKindF16, 1)
RB_INST_MAJORS(kKindF16, 2)
RB_INST_MAJORS(kKindI8, 1)
RB_INST_MAJORS(kKindI8, 2)
RB_INST_MAJORS(kKindF8, 1)
RB_INST_MAJORS(kKindF8, 2)
RB_INST(kKindTF32, false, false, 1)
RB_INST(kKindTF32, false, false, 2)
}  // namespace rb
