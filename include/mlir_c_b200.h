/* The MLIR C API surface that MIGraphX drives rocMLIR through, served by the B200 kernel library.
 *
 * rocMLIR's production client builds a `func.func` of `migraphx.*` ops with the generic MLIR C builder calls, runs
 * three pipelines on it and reads back {kernel info, block/grid, code object}
 * (mlir/include/mlir-c/Dialect/MIGraphX.h:27-78, mlir/include/mlir-c/Dialect/Rock.h:22-166; the call sequence is
 * mlir/test/CAPI/mixr_full.c:30-347). This header keeps those names, argument meanings and return conventions, so
 * that such a client compiles and links against librocmlir_b200.so unchanged in its own code:
 *
 *  - the generic builder subset the client uses (contexts, locations, types, attributes, operation states, blocks,
 *    regions, modules, pass managers: mlir-c/IR.h, mlir-c/Pass.h, mlir-c/BuiltinTypes.h, mlir-c/BuiltinAttributes.h of
 *    external/llvm-project) is backed by a small operation graph, not by MLIR: operations are kept as built, nothing
 *    is verified until a pipeline runs;
 *  - mlirModuleCreateParse reads the textual form of the same graphs (the files under mlir/test/fusion/pr-e2e);
 *  - mlirMIGraphXAddHighLevelPipeline recognises the contraction (migraphx.dot / quant_dot / convolution /
 *    quant_convolution) with the elementwise tail this library fuses (broadcast and same-shape adds, relu, clip,
 *    dequantizelinear, quantizelinear, convert, scalar mul) and fails - the reference's "not applicable", never a
 *    crash - on anything else; ...AddApplicabilityPipeline checks the tile configuration a perf_config asks for;
 *    ...AddBackendPipeline(pm, arch) accepts `sm_100a` (false for any other architecture, AMD names included) and
 *    fixes the launch geometry;
 *  - mlirGetKernelInfo / mlirGetKernelAttrs / mlirGetBinary answer in the reference's formats; the binary is the
 *    library's sm_100a cubin, and rbModuleGetKernelLaunch adds what two integers cannot carry (see RbKernelLaunch);
 *  - the tuning entry points mlirRockTuning*, mlirIsSplitKFaster, mlirIsModuleFusible, mlirGetNumPrefillArgs,
 *    mlirGetNumAuxBuffers take the module, like the reference's.
 *
 * Kernel calling convention (mlir/lib/Dialect/Rock/Pipelines/Pipelines.cpp:138,246-248): bare device pointers in
 * function-argument order, results last. rbModuleLaunch takes them in that order. */
#ifndef MLIR_C_B200_H
#define MLIR_C_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "rocmlir_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MLIR_CAPI_EXPORTED RB_EXPORT

/* mlir-c/Dialect/MIGraphX.h:26 and mlir-c/Dialect/Rock.h:22 */
#define MLIR_MIGRAPHX_DIALECT_API_VERSION 4
#define MLIR_ROCK_C_API_VERSION 2

/* mlir-c/IR.h:50-66, mlir-c/Pass.h, mlir-c/Support.h: one-pointer handle structs */
typedef struct MlirContext { void *ptr; } MlirContext;
typedef struct MlirLocation { const void *ptr; } MlirLocation;
typedef struct MlirModule { const void *ptr; } MlirModule;
typedef struct MlirOperation { void *ptr; } MlirOperation;
typedef struct MlirBlock { void *ptr; } MlirBlock;
typedef struct MlirRegion { void *ptr; } MlirRegion;
typedef struct MlirValue { const void *ptr; } MlirValue;
typedef struct MlirType { const void *ptr; } MlirType;
typedef struct MlirAttribute { const void *ptr; } MlirAttribute;
typedef struct MlirIdentifier { const void *ptr; } MlirIdentifier;
typedef struct MlirPassManager { void *ptr; } MlirPassManager;
typedef struct MlirStringRef { const char *data; size_t length; } MlirStringRef;
typedef struct MlirLogicalResult { int8_t value; } MlirLogicalResult;
typedef struct MlirNamedAttribute { MlirIdentifier name; MlirAttribute attribute; } MlirNamedAttribute;

static inline MlirStringRef mlirStringRefCreate(const char *str, size_t length) { MlirStringRef r = {str, length}; return r; }
MLIR_CAPI_EXPORTED MlirStringRef mlirStringRefCreateFromCString(const char *str);
static inline bool mlirLogicalResultIsSuccess(MlirLogicalResult res) { return res.value != 0; }
static inline bool mlirLogicalResultIsFailure(MlirLogicalResult res) { return res.value == 0; }
static inline bool mlirModuleIsNull(MlirModule m) { return !m.ptr; }
static inline bool mlirAttributeIsNull(MlirAttribute a) { return !a.ptr; }
static inline bool mlirTypeIsNull(MlirType t) { return !t.ptr; }

/* mlir-c/IR.h:330-346 */
typedef struct MlirOperationState {
  MlirStringRef name;
  MlirLocation location;
  intptr_t nResults;
  MlirType *results;
  intptr_t nOperands;
  MlirValue *operands;
  intptr_t nRegions;
  MlirRegion *regions;
  intptr_t nSuccessors;
  MlirBlock *successors;
  intptr_t nAttributes;
  MlirNamedAttribute *attributes;
  bool enableResultTypeInference;
} MlirOperationState;

/* ---- context, location ------------------------------------------------------------------------------------------ */
MLIR_CAPI_EXPORTED MlirContext mlirContextCreate(void);
MLIR_CAPI_EXPORTED void mlirContextDestroy(MlirContext context);   /* frees everything built in the context */
MLIR_CAPI_EXPORTED MlirLocation mlirLocationUnknownGet(MlirContext context);

/* ---- types (mlir-c/BuiltinTypes.h; MIGraphX.h:32-43) ----------------------------------------------------------------- */
MLIR_CAPI_EXPORTED MlirType mlirF32TypeGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirType mlirF16TypeGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirType mlirBF16TypeGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirType mlirFloat8E4M3FNTypeGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirType mlirFloat8E5M2TypeGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirType mlirIntegerTypeGet(MlirContext ctx, unsigned bitwidth);
MLIR_CAPI_EXPORTED MlirType mlirTypeParseGet(MlirContext ctx, MlirStringRef type);
MLIR_CAPI_EXPORTED MlirType rocmlirMIXRShapedTypeGet(intptr_t rank, const int64_t *shape, const int64_t *strides,
                                                     MlirType elementType);
MLIR_CAPI_EXPORTED bool rocmlirIsAMIXRShapedType(MlirType type);
MLIR_CAPI_EXPORTED MlirType rocmlirMIXRShapedTypeAsTensor(MlirType type);

/* ---- attributes (mlir-c/BuiltinAttributes.h, IR.h) -------------------------------------------------------------------- */
MLIR_CAPI_EXPORTED MlirAttribute mlirAttributeParseGet(MlirContext ctx, MlirStringRef attr);   /* null on a parse error */
MLIR_CAPI_EXPORTED MlirAttribute mlirUnitAttrGet(MlirContext ctx);
MLIR_CAPI_EXPORTED MlirAttribute mlirStringAttrGet(MlirContext ctx, MlirStringRef str);
MLIR_CAPI_EXPORTED MlirAttribute mlirIntegerAttrGet(MlirType type, int64_t value);
MLIR_CAPI_EXPORTED MlirIdentifier mlirIdentifierGet(MlirContext ctx, MlirStringRef str);
MLIR_CAPI_EXPORTED MlirNamedAttribute mlirNamedAttributeGet(MlirIdentifier name, MlirAttribute attr);

/* ---- modules, regions, blocks, operations ------------------------------------------------------------------------------ */
MLIR_CAPI_EXPORTED MlirModule mlirModuleCreateEmpty(MlirLocation location);
MLIR_CAPI_EXPORTED MlirModule mlirModuleCreateParse(MlirContext ctx, MlirStringRef module);   /* null on a parse error */
MLIR_CAPI_EXPORTED MlirBlock mlirModuleGetBody(MlirModule module);
MLIR_CAPI_EXPORTED MlirOperation mlirModuleGetOperation(MlirModule module);
MLIR_CAPI_EXPORTED MlirModule mlirModuleFromOperation(MlirOperation op);
MLIR_CAPI_EXPORTED void mlirModuleDestroy(MlirModule module);
MLIR_CAPI_EXPORTED MlirRegion mlirRegionCreate(void);
MLIR_CAPI_EXPORTED void mlirRegionAppendOwnedBlock(MlirRegion region, MlirBlock block);
MLIR_CAPI_EXPORTED MlirBlock mlirBlockCreate(intptr_t nArgs, MlirType const *args, MlirLocation const *locs);
MLIR_CAPI_EXPORTED MlirValue mlirBlockGetArgument(MlirBlock block, intptr_t pos);
MLIR_CAPI_EXPORTED void mlirBlockAppendOwnedOperation(MlirBlock block, MlirOperation operation);
MLIR_CAPI_EXPORTED void mlirBlockInsertOwnedOperation(MlirBlock block, intptr_t pos, MlirOperation operation);
MLIR_CAPI_EXPORTED MlirOperationState mlirOperationStateGet(MlirStringRef name, MlirLocation loc);
MLIR_CAPI_EXPORTED void mlirOperationStateAddResults(MlirOperationState *state, intptr_t n, MlirType const *results);
MLIR_CAPI_EXPORTED void mlirOperationStateAddOperands(MlirOperationState *state, intptr_t n, MlirValue const *operands);
MLIR_CAPI_EXPORTED void mlirOperationStateAddOwnedRegions(MlirOperationState *state, intptr_t n, MlirRegion const *regions);
MLIR_CAPI_EXPORTED void mlirOperationStateAddAttributes(MlirOperationState *state, intptr_t n,
                                                        MlirNamedAttribute const *attributes);
MLIR_CAPI_EXPORTED MlirOperation mlirOperationCreate(MlirOperationState *state);
MLIR_CAPI_EXPORTED MlirOperation mlirOperationClone(MlirOperation op);
MLIR_CAPI_EXPORTED void mlirOperationSetAttributeByName(MlirOperation op, MlirStringRef name, MlirAttribute attr);
MLIR_CAPI_EXPORTED MlirValue mlirOperationGetResult(MlirOperation op, intptr_t pos);
MLIR_CAPI_EXPORTED void mlirOperationDump(MlirOperation op);   /* the generic textual form, to stderr */

/* ---- pass managers (mlir-c/Pass.h) and the three pipelines (MIGraphX.h:60-78) ---------------------------------------------- */
MLIR_CAPI_EXPORTED MlirPassManager mlirPassManagerCreate(MlirContext ctx);
MLIR_CAPI_EXPORTED void mlirPassManagerDestroy(MlirPassManager passManager);
MLIR_CAPI_EXPORTED MlirLogicalResult mlirPassManagerRunOnOp(MlirPassManager passManager, MlirOperation op);
MLIR_CAPI_EXPORTED void mlirMIGraphXAddHighLevelPipeline(MlirPassManager pm);
MLIR_CAPI_EXPORTED void mlirMIGraphXAddApplicabilityPipeline(MlirPassManager pm);
MLIR_CAPI_EXPORTED bool mlirMIGraphXAddBackendPipeline(MlirPassManager pm, const char *arch);

/* ---- what the client reads back (MIGraphX.h:45-56; blob format mlir/lib/CAPI/Dialect/MIGraphX.cpp:54-90) --------------------- */
/* Blob: int32[1 + nargs + sum(rank)] = {nargs, rank_0, dims_0..., rank_1, ...} followed by the kernel name's bytes (no
 * terminator); arguments are the function's arguments then its results; the dimensions are those of each tensor as
 * laid out in memory (sorted by stride). data == NULL: *size receives the byte count. */
MLIR_CAPI_EXPORTED void mlirGetKernelInfo(MlirModule module, int *size, void *data);
/* attrs[0] = block size, attrs[1] = grid size (1-D launch) of the module's kernel; needs the backend pipeline. */
MLIR_CAPI_EXPORTED void mlirGetKernelAttrs(MlirModule module, uint32_t *attrs);
/* Two-call protocol like the reference: bin == NULL gives the size. The image is the library's sm_100a cubin. False
 * before the backend pipeline has run, or when both pointers are NULL. */
MLIR_CAPI_EXPORTED bool mlirGetBinary(MlirModule module, size_t *size, char *bin);

/* ---- beyond the reference's three getters -------------------------------------------------------------------------------- */
/* Launch description for a client that loads the cubin itself: args = device pointers in kernel-argument order (the
 * function's arguments, then its result). RB_UNSUPPORTED when the module runs as several kernels. */
MLIR_CAPI_EXPORTED RbStatus rbModuleGetKernelLaunch(MlirModule module, void *const *args, size_t nargs, RbKernelLaunch *out);
/* Device workspace the module's launch needs, and the launch itself through the library's own launcher. */
MLIR_CAPI_EXPORTED size_t rbModuleGetWorkspaceSize(MlirModule module);
MLIR_CAPI_EXPORTED RbStatus rbModuleLaunch(MlirModule module, void *const *args, size_t nargs, void *workspace,
                                           size_t workspace_bytes, void *stream);
/* Why the last pipeline run on this module failed ("" if it did not): the reference prints diagnostics to stderr. */
MLIR_CAPI_EXPORTED const char *rbModuleGetDiagnostic(MlirModule module);

/* ---- tuning (Rock.h:26-166) ------------------------------------------------------------------------------------------------- */
typedef enum RocmlirTuningParamSetKind {   /* mlir-c/Dialect/RockEnums.h:18-22 */
  RocmlirTuningParamSetKindQuick = 0,
  RocmlirTuningParamSetKindFull = 1,
  RocmlirTuningParamSetKindExhaustive = 2
} RocmlirTuningParamSetKind;
enum RocmlirSplitKSelectionLikelihood { never = 0, maybe = 1, always = 2 };   /* RockEnums.h:24-27 */
typedef struct MlirRockTuningSpace { void *ptr; } MlirRockTuningSpace;
typedef struct MlirRockTuningParam { void *ptr; } MlirRockTuningParam;
typedef struct MlirRockTuningTable { void *ptr; } MlirRockTuningTable;
#define ROCMLIR_TUNING_PARAM_STRING_BUFSZ 64
#define ROCMLIR_TUNING_KEY_BUFSZ 2048
MLIR_CAPI_EXPORTED MlirRockTuningSpace mlirRockTuningSpaceCreate(MlirModule module, RocmlirTuningParamSetKind kind);
MLIR_CAPI_EXPORTED unsigned mlirRockTuningGetNumParams(MlirRockTuningSpace params);
MLIR_CAPI_EXPORTED MlirRockTuningParam mlirRockTuningParamCreate(void);
MLIR_CAPI_EXPORTED void mlirRockTuningParamDestroy(MlirRockTuningParam param);
MLIR_CAPI_EXPORTED void mlirRockTuningSpaceDestroy(MlirRockTuningSpace params);
MLIR_CAPI_EXPORTED bool mlirRockTuningParamGet(MlirRockTuningSpace params, unsigned pos, MlirRockTuningParam param);
MLIR_CAPI_EXPORTED bool mlirRockTuningParamGetQuick(MlirRockTuningSpace params, unsigned pos, MlirRockTuningParam param);
MLIR_CAPI_EXPORTED size_t mlirRockTuningParamToString(MlirRockTuningParam param, char *buf, size_t bufLen);
MLIR_CAPI_EXPORTED bool mlirRockTuningSetParam(MlirModule module, MlirRockTuningParam param);
MLIR_CAPI_EXPORTED bool mlirRockTuningSetFromStr(MlirModule module, MlirStringRef perfStr);
MLIR_CAPI_EXPORTED MlirRockTuningTable mlirRockTuningTableCreate(void);
MLIR_CAPI_EXPORTED void mlirRockTuningTableDestroy(MlirRockTuningTable table);
MLIR_CAPI_EXPORTED bool mlirRockTuningUpdateTable(MlirRockTuningTable perfTable, MlirStringRef problemKey,
                                                  MlirStringRef perfStr, float time);
MLIR_CAPI_EXPORTED bool mlirRockTuningSetFromTable(MlirRockTuningTable perfTable, MlirModule module);
MLIR_CAPI_EXPORTED size_t mlirRockTuningGetKey(MlirModule module, char *buf, size_t bufLen);
MLIR_CAPI_EXPORTED enum RocmlirSplitKSelectionLikelihood mlirIsSplitKFaster(int64_t gDim, int64_t mDim, int64_t nDim,
                                                                            int64_t kDim, int64_t numCUs,
                                                                            RocmlirTuningParamSetKind tuningLevel);
MLIR_CAPI_EXPORTED bool mlirIsModuleFusible(MlirModule module, MlirStringRef perfStr);
MLIR_CAPI_EXPORTED size_t mlirGetNumPrefillArgs(MlirModule module);
MLIR_CAPI_EXPORTED void mlirGetPrefillArgsInfo(MlirModule module, size_t *indices, MlirAttribute *initValues, size_t length);
MLIR_CAPI_EXPORTED size_t mlirGetNumAuxBuffers(MlirModule module);
MLIR_CAPI_EXPORTED void mlirGetAuxBuffersInfo(MlirModule module, size_t *sizes, MlirAttribute *initValues, size_t length);

#ifdef __cplusplus
}
#endif
#endif /* MLIR_C_B200_H */
