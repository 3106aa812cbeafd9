/* Tuning surface of rocmlir_b200: the counterpart of rocMLIR's mlir-c tuning API
 * (mlir/include/mlir-c/Dialect/Rock.h:39-166, implementation mlir/lib/CAPI/Dialect/Rock.cpp:31-205 and
 * mlir/lib/Dialect/Rock/Tuning/RockTuningImpl.cpp). The reference's functions take an MlirModule holding one
 * rock.gemm / rock.conv* / rock.attention; here the same role is played by an RbProblem created from an option
 * string (the grammar of include/miir_b200.h) or from a problem struct. Names, return conventions and buffer
 * semantics follow the reference function named beside each declaration.
 */
#ifndef ROCMLIR_B200_TUNING_H
#define ROCMLIR_B200_TUNING_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "rocmlir_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Rock.h:22 MLIR_ROCK_C_API_VERSION */
#define RB_TUNING_API_VERSION 2

/* mlir-c/Dialect/RockEnums.h:18-27 */
typedef enum RbTuningParamSetKind {
  RbTuningParamSetKindQuick = 0,
  RbTuningParamSetKindFull = 1,
  RbTuningParamSetKindExhaustive = 2
} RbTuningParamSetKind;
typedef enum RbSplitKSelectionLikelihood { RbSplitKNever = 0, RbSplitKMaybe = 1, RbSplitKAlways = 2 } RbSplitKSelectionLikelihood;

/* Opaque handles, one pointer each as in Rock.h:26-36. */
typedef struct RbProblem { void *ptr; } RbProblem;
typedef struct RbTuningSpace { void *ptr; } RbTuningSpace;
typedef struct RbTuningParam { void *ptr; } RbTuningParam;
typedef struct RbTuningTable { void *ptr; } RbTuningTable;

/* The "module": one problem of the path. ptr == NULL on failure (bad options / no kernel for the problem). */
RB_EXPORT RbProblem rbProblemCreate(const char *options);
RB_EXPORT RbProblem rbProblemFromGemm(const RbGemmProblem *p);
RB_EXPORT RbProblem rbProblemFromConv(const RbConvProblem *p);
RB_EXPORT RbProblem rbProblemFromAttention(const RbAttentionProblem *p);
RB_EXPORT void rbProblemDestroy(RbProblem problem);
/* The perf_config currently attached ("" = the library's own choice) and the variant word it stands for. */
RB_EXPORT size_t rbProblemGetPerfConfig(RbProblem problem, char *buf, size_t bufLen);
RB_EXPORT uint32_t rbProblemGetVariant(RbProblem problem);

/* mlirRockTuningSpaceCreate (Rock.h:39): the configurations worth measuring for the problem. Quick = the
 * library's choice and its nearest alternatives; Full = every tile shape x K split x stream-K setting that is
 * valid for the problem; Exhaustive = Full x every ring depth. */
RB_EXPORT RbTuningSpace rbTuningSpaceCreate(RbProblem problem, RbTuningParamSetKind kind);
/* mlirRockTuningGetNumParams (Rock.h:43) */
RB_EXPORT unsigned rbTuningGetNumParams(RbTuningSpace space);
/* mlirRockTuningParamCreate / Destroy / SpaceDestroy (Rock.h:46-54) */
RB_EXPORT RbTuningParam rbTuningParamCreate(void);
RB_EXPORT void rbTuningParamDestroy(RbTuningParam param);
RB_EXPORT void rbTuningSpaceDestroy(RbTuningSpace space);
/* mlirRockTuningParamGet (Rock.h:59): copies entry `pos` into `param`; false when pos is out of range. */
RB_EXPORT bool rbTuningParamGet(RbTuningSpace space, unsigned pos, RbTuningParam param);
/* mlirRockTuningParamGetQuick (Rock.h:66; declared by the reference but defined nowhere in its tree): entry `pos`
 * of the quick set of the space's problem, whatever kind the space was created with. */
RB_EXPORT bool rbTuningParamGetQuick(RbTuningSpace space, unsigned pos, RbTuningParam param);

/* Rock.h:70 */
#define RB_TUNING_PARAM_STRING_BUFSZ 64
/* mlirRockTuningParamToString (Rock.h:80): strncpy semantics - returns the true length, and leaves the buffer
 * unterminated when it is too small. */
RB_EXPORT size_t rbTuningParamToString(RbTuningParam param, char *buf, size_t bufLen);
/* mlirRockTuningSetParam / SetFromStr (Rock.h:84-89): false when the configuration is not valid for the problem. */
RB_EXPORT bool rbTuningSetParam(RbProblem problem, RbTuningParam param);
RB_EXPORT bool rbTuningSetFromStr(RbProblem problem, const char *perfStr, size_t perfLen);

/* mlirRockTuningTableCreate / Destroy (Rock.h:94-99). A table may be shared between threads (readers-writer lock,
 * as mlir/include/mlir/Dialect/Rock/Tuning/RockTuning.h:58-65). */
RB_EXPORT RbTuningTable rbTuningTableCreate(void);
RB_EXPORT void rbTuningTableDestroy(RbTuningTable table);
/* mlirRockTuningUpdateTable (Rock.h:108): keeps only the fastest entry per key; true if the table changed. */
RB_EXPORT bool rbTuningUpdateTable(RbTuningTable table, const char *problemKey, size_t keyLen, const char *perfStr,
                                   size_t perfLen, float time);
/* mlirRockTuningSetFromTable (Rock.h:116): false when the table has no entry for the problem's key. */
RB_EXPORT bool rbTuningSetFromTable(RbTuningTable table, RbProblem problem);

/* The tuning database in the reference's text form (mlir/utils/performance/tuningRunner.py:393-404, read by
 * perfRunner.py:174-200): `arch <tab> numCUs <tab> problem <tab> perf_config [<tab> TFlops]`, or the legacy
 * `arch <tab> problem <tab> perf_config`; '#' starts a comment. `arch <tab> numCUs <tab> problem` is exactly the key
 * rbTuningGetKey returns. Load returns the number of entries taken, Save the number written, -1 when the file
 * cannot be opened. */
RB_EXPORT int rbTuningTableLoad(RbTuningTable table, const char *path);
RB_EXPORT int rbTuningTableSave(RbTuningTable table, const char *path, const char *space_name);

/* Process-wide database: every launch whose variant word is 0 (rbSetGemmVariant) looks its problem key up here and
 * runs the recorded configuration; workspace queries follow the same rule, so sizes and launches agree. At first
 * use the library loads the file named by the environment variable RB_TUNING_DB ("none" or empty: no database), or,
 * when the variable is unset, tuned/sm_100a.tsv beside the shared library (the measured table this package ships;
 * written by the rocmlir-tuning-driver tool). Rows of other architectures and perf_config strings this library
 * cannot map are skipped. rbTuningDbLoad adds a file's rows (returns the number taken, -1 = cannot open). */
RB_EXPORT int rbTuningDbLoad(const char *path);
RB_EXPORT void rbTuningDbClear(void);
RB_EXPORT int rbTuningDbSize(void);
RB_EXPORT uint32_t rbTuningDbLookup(RbProblem problem); /* variant word recorded for the problem, 0 = none */

/* Rock.h:120 */
#define RB_TUNING_KEY_BUFSZ 2048
/* mlirRockTuningGetKey (Rock.h:133): "<arch>\t<numCU>\t<problem flags>" in the reference's format
 * (RockTuningImpl.cpp:550-876), strncpy semantics, (size_t)-1 when no key can be formed. */
RB_EXPORT size_t rbTuningGetKey(RbProblem problem, char *buf, size_t bufLen);

/* mlirIsSplitKFaster (Rock.h:139, RockTuningImpl.cpp:962-1008): same decision procedure (work imbalance of the
 * data-parallel launch over every tile shape; thresholds 1.20 / 1.30 / 1.80; split factors 3 and 4; Quick never
 * splits) over this library's tile shapes. */
RB_EXPORT RbSplitKSelectionLikelihood rbIsSplitKFaster(int64_t gDim, int64_t mDim, int64_t nDim, int64_t kDim,
                                                       int64_t numCUs, RbTuningParamSetKind tuningLevel);
/* mlirIsModuleFusible (Rock.h:144): whether fused elementwise work stays legal under `perfStr`. Always true here:
 * a K split keeps f32 planes and its reduction kernel applies the epilogue (the reference must refuse fusions
 * that atomic adds would break, RockTuningImpl.cpp:1010-1015). False only for a malformed string. */
RB_EXPORT bool rbIsProblemFusible(RbProblem problem, const char *perfStr, size_t perfLen);
/* mlirGetNumPrefillArgs (Rock.h:149): output buffers the caller must pre-fill before the launch. Always 0:
 * no kernel of this library accumulates into its output with atomics. */
RB_EXPORT size_t rbGetNumPrefillArgs(RbProblem problem);
/* mlirGetNumAuxBuffers (Rock.h:159; always 0 in the reference too, mlir/lib/CAPI/Dialect/Rock.cpp:201-205). */
RB_EXPORT size_t rbGetNumAuxBuffers(RbProblem problem);

#ifdef __cplusplus
}
#endif
#endif /* ROCMLIR_B200_TUNING_H */
