/* The call sequence of rocMLIR's own C-API example (mlir/test/CAPI/mixr_full.c:30-347) against this library's header:
 * build   func @main(%in, %filter, %bias) = relu(convolution(%in, %filter) + broadcast(%bias))   with the generic
 * builder calls, run the high-level pipeline, walk the tuning space on clones with the applicability pipeline, record
 * times in a tuning table, set the best entry, read the kernel info blob, run the backend pipeline, read block / grid
 * and the binary. No GPU is needed: everything up to and including mlirGetBinary is host work.
 *   cc -I include -o mlirc_client mlirc_client.c -ldl ; ./mlirc_client librocmlir_b200.so */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "mlir_c_b200.h"

static MlirNamedAttribute named(MlirContext ctx, const char *name, const char *text) {
  return mlirNamedAttributeGet(mlirIdentifierGet(ctx, mlirStringRefCreateFromCString(name)),
                               mlirAttributeParseGet(ctx, mlirStringRefCreateFromCString(text)));
}

static MlirModule make_conv_bias_relu(MlirContext ctx, MlirLocation loc) {
  MlirModule module = mlirModuleCreateEmpty(loc);
  MlirBlock moduleBody = mlirModuleGetBody(module);
  int64_t inDims[] = {1, 64, 56, 56}, inStrides[] = {200704, 3136, 56, 1};
  int64_t filDims[] = {64, 64, 1, 1}, filStrides[] = {64, 1, 1, 1};
  int64_t biasDims[] = {64}, biasStrides[] = {1};
  int64_t bcastStrides[] = {0, 1, 0, 0};
  MlirType f32 = mlirF32TypeGet(ctx);
  MlirType inType = rocmlirMIXRShapedTypeGet(4, inDims, inStrides, f32);
  MlirType filType = rocmlirMIXRShapedTypeGet(4, filDims, filStrides, f32);
  MlirType biasType = rocmlirMIXRShapedTypeGet(1, biasDims, biasStrides, f32);
  MlirType bcastType = rocmlirMIXRShapedTypeGet(4, inDims, bcastStrides, f32);
  MlirType argTypes[] = {inType, filType, biasType};
  MlirLocation locs[] = {loc, loc, loc};
  MlirRegion region = mlirRegionCreate();
  MlirBlock body = mlirBlockCreate(3, argTypes, locs);
  mlirRegionAppendOwnedBlock(region, body);

  MlirNamedAttribute funcAttrs[] = {
      named(ctx, "function_type",
            "(!migraphx.shaped<1x64x56x56xf32, 200704x3136x56x1>, !migraphx.shaped<64x64x1x1xf32, 64x1x1x1>, "
            "!migraphx.shaped<64xf32, 1>) -> (!migraphx.shaped<1x64x56x56xf32, 200704x3136x56x1>)"),
      named(ctx, "sym_name", "\"main\"")};
  MlirOperationState funcState = mlirOperationStateGet(mlirStringRefCreateFromCString("func.func"), loc);
  mlirOperationStateAddAttributes(&funcState, 2, funcAttrs);
  mlirOperationStateAddOwnedRegions(&funcState, 1, &region);
  MlirOperation func = mlirOperationCreate(&funcState);
  mlirOperationSetAttributeByName(func, mlirStringRefCreateFromCString("kernel"), mlirUnitAttrGet(ctx));
  mlirOperationSetAttributeByName(func, mlirStringRefCreateFromCString("arch"),
                                  mlirStringAttrGet(ctx, mlirStringRefCreateFromCString("sm_100a")));
  mlirBlockInsertOwnedOperation(moduleBody, 0, func);

  MlirValue convOperands[] = {mlirBlockGetArgument(body, 0), mlirBlockGetArgument(body, 1)};
  MlirNamedAttribute convAttrs[] = {named(ctx, "padding", "[0:i64, 0:i64, 0:i64, 0:i64]"), named(ctx, "stride", "[1:i64, 1:i64]"),
                                    named(ctx, "dilation", "[1:i64, 1:i64]"), named(ctx, "group", "1:i64"),
                                    named(ctx, "padding_mode", "0:i64")};
  MlirOperationState convState = mlirOperationStateGet(mlirStringRefCreateFromCString("migraphx.convolution"), loc);
  mlirOperationStateAddResults(&convState, 1, &inType);
  mlirOperationStateAddOperands(&convState, 2, convOperands);
  mlirOperationStateAddAttributes(&convState, 5, convAttrs);
  MlirOperation conv = mlirOperationCreate(&convState);
  mlirBlockAppendOwnedOperation(body, conv);

  MlirValue biasArg = mlirBlockGetArgument(body, 2);
  MlirNamedAttribute bcastAttrs[] = {named(ctx, "axis", "1:i64"), named(ctx, "out_lens", "[1:i64, 64:i64, 56:i64, 56:i64]")};
  MlirOperationState bcastState = mlirOperationStateGet(mlirStringRefCreateFromCString("migraphx.broadcast"), loc);
  mlirOperationStateAddResults(&bcastState, 1, &bcastType);
  mlirOperationStateAddOperands(&bcastState, 1, &biasArg);
  mlirOperationStateAddAttributes(&bcastState, 2, bcastAttrs);
  MlirOperation bcast = mlirOperationCreate(&bcastState);
  mlirBlockAppendOwnedOperation(body, bcast);

  MlirValue addOperands[] = {mlirOperationGetResult(conv, 0), mlirOperationGetResult(bcast, 0)};
  MlirOperationState addState = mlirOperationStateGet(mlirStringRefCreateFromCString("migraphx.add"), loc);
  mlirOperationStateAddResults(&addState, 1, &inType);
  mlirOperationStateAddOperands(&addState, 2, addOperands);
  MlirOperation add = mlirOperationCreate(&addState);
  mlirBlockAppendOwnedOperation(body, add);

  MlirValue reluOperand = mlirOperationGetResult(add, 0);
  MlirOperationState reluState = mlirOperationStateGet(mlirStringRefCreateFromCString("migraphx.relu"), loc);
  mlirOperationStateAddResults(&reluState, 1, &inType);
  mlirOperationStateAddOperands(&reluState, 1, &reluOperand);
  MlirOperation relu = mlirOperationCreate(&reluState);
  mlirBlockAppendOwnedOperation(body, relu);

  MlirValue retOperand = mlirOperationGetResult(relu, 0);
  MlirOperationState retState = mlirOperationStateGet(mlirStringRefCreateFromCString("func.return"), loc);
  mlirOperationStateAddOperands(&retState, 1, &retOperand);
  mlirBlockAppendOwnedOperation(body, mlirOperationCreate(&retState));
  return module;
}

int main(void) {
  MlirContext ctx = mlirContextCreate();
  MlirLocation loc = mlirLocationUnknownGet(ctx);
  MlirModule module = make_conv_bias_relu(ctx, loc);
  MlirOperation moduleOp = mlirModuleGetOperation(module);
  MlirPassManager highLevelPm = mlirPassManagerCreate(ctx), applicabilityPm = mlirPassManagerCreate(ctx),
                  backendPm = mlirPassManagerCreate(ctx);
  mlirMIGraphXAddHighLevelPipeline(highLevelPm);
  if (mlirLogicalResultIsFailure(mlirPassManagerRunOnOp(highLevelPm, moduleOp))) {
    printf("Running high-level pipeline failed: %s\n", rbModuleGetDiagnostic(module));
    return 1;
  }
  MlirRockTuningSpace space = mlirRockTuningSpaceCreate(module, RocmlirTuningParamSetKindFull);
  unsigned fNum = mlirRockTuningGetNumParams(space);
  printf("full set = %u\n", fNum);
  MlirRockTuningParam param = mlirRockTuningParamCreate();
  MlirRockTuningTable table = mlirRockTuningTableCreate();
  mlirMIGraphXAddApplicabilityPipeline(applicabilityPm);
  char key[ROCMLIR_TUNING_KEY_BUFSZ];
  size_t keyBytes = mlirRockTuningGetKey(module, key, ROCMLIR_TUNING_KEY_BUFSZ);
  if (keyBytes >= ROCMLIR_TUNING_KEY_BUFSZ) return 1;
  key[keyBytes] = 0;
  printf("problem key: %s\n", key);
  unsigned successes = 0;
  for (unsigned i = 0; i < fNum && successes < 2; ++i) {
    if (!mlirRockTuningParamGet(space, i, param)) { printf("fails to obtain param\n"); return 1; }
    char paramStr[ROCMLIR_TUNING_PARAM_STRING_BUFSZ];
    size_t n = mlirRockTuningParamToString(param, paramStr, ROCMLIR_TUNING_PARAM_STRING_BUFSZ);
    if (n >= ROCMLIR_TUNING_PARAM_STRING_BUFSZ) return 1;
    paramStr[n] = 0;
    MlirModule clone = mlirModuleFromOperation(mlirOperationClone(mlirModuleGetOperation(module)));
    mlirRockTuningSetParam(clone, param);
    if (mlirLogicalResultIsFailure(mlirPassManagerRunOnOp(applicabilityPm, mlirModuleGetOperation(clone)))) {
      printf("Perfconfig \"%s\" is not applicable\n", paramStr);
      mlirModuleDestroy(clone);
      continue;
    }
    printf("Update perfconfig: \"%s\" with time %f\n", paramStr, (float)(i + 1));
    if (!mlirRockTuningUpdateTable(table, mlirStringRefCreateFromCString(key), mlirStringRefCreateFromCString(paramStr), (float)(i + 1)))
      printf("fails to update table, existing config is faster\n");
    ++successes;
    mlirModuleDestroy(clone);
  }
  if (!mlirRockTuningSetFromTable(table, module)) { printf("fails to set param\n"); return 1; }
  mlirRockTuningTableDestroy(table);
  mlirRockTuningParamDestroy(param);
  mlirRockTuningSpaceDestroy(space);

  int argSize = 0;
  mlirGetKernelInfo(module, &argSize, NULL);
  void *argInfo = malloc(argSize + 1);
  mlirGetKernelInfo(module, NULL, argInfo);
  int *argData = (int *)argInfo, idx = 1;
  for (int i = 0; i < argData[0]; i++) {
    int rank = argData[idx++];
    printf("%d:<", rank);
    for (int j = 0; j < rank; j++) printf("%s%d", j ? "," : "", argData[idx++]);
    printf("> ");
  }
  ((char *)argInfo)[argSize] = '\0';
  printf("\nkernel name : %s\n", (char *)(argData + idx));

  if (mlirMIGraphXAddBackendPipeline(backendPm, "gfx908:sramecc+:xnack-")) { printf("an AMD architecture was accepted\n"); return 1; }
  if (!mlirMIGraphXAddBackendPipeline(backendPm, "sm_100a")) { printf("Errors in building backend pipeline\n"); return 1; }
  if (mlirLogicalResultIsFailure(mlirPassManagerRunOnOp(backendPm, moduleOp))) {
    printf("Errors in running backend pipeline: %s\n", rbModuleGetDiagnostic(module));
    return 1;
  }
  uint32_t attrs[2];
  mlirGetKernelAttrs(module, attrs);
  printf("block size : %u, grid size : %u\n", attrs[0], attrs[1]);
  size_t binSize = 0;
  if (!mlirGetBinary(module, &binSize, NULL)) return 1;
  char *bin = malloc(binSize);
  if (!mlirGetBinary(module, NULL, bin)) return 1;
  printf("bin size : %zu, magic %02x %c%c%c\n", binSize, (unsigned char)bin[0], bin[1], bin[2], bin[3]);
  printf("workspace : %zu\n", rbModuleGetWorkspaceSize(module));
  printf("PASSED!\n");
  mlirPassManagerDestroy(highLevelPm); mlirPassManagerDestroy(applicabilityPm); mlirPassManagerDestroy(backendPm);
  mlirModuleDestroy(module);
  mlirContextDestroy(ctx);
  return 0;
}
