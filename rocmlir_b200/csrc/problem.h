// A problem of the path as the string-configured entry points see it: parsed from the reference's option grammar
// (mlir/lib/Dialect/Rock/Generator/ConvGenerator.cpp:82-98,487-668 for convolutions; rocmlir-gen's flag names for
// gemm and attention), validated the way ConvGenerator::isApplicable does (:139-245), with the tile configuration
// an optional perf_config selects.
#pragma once
#include <stdint.h>

#include <string>

#include "../../include/rocmlir_b200.h"

namespace rb {

enum ProblemKind : uint32_t { kConv = 1, kGemm = 2, kAttention = 3 };

struct ProblemDesc {
  uint32_t kind = 0;
  uint32_t variant = 0;     // rbSetGemmVariant word from perf_config (0 = the library chooses)
  size_t workspace = 0;     // bytes of device workspace under that variant
  RbConvProblem conv;
  RbGemmProblem gemm;
  RbAttentionProblem att;
  std::string arch, kernel_name, perf_config;
  int num_cu = 0;
  int kernel_id = -1;
};

// False when a required key is missing, a value is malformed, the dimensions are inconsistent, the architecture
// is not this one, or the library has no kernel for the problem.
bool parse_problem(const char* options, ProblemDesc* out);

// Recomputes `workspace` after `variant` changed. False if the variant is not usable for the problem.
bool refresh_problem(ProblemDesc* d);

// perf_config strings of this library: "b200:<tile_m>,<tile_n>,<stages>,<splitK>,<streamK>[,<kpr>]" with tile_m 128
// (one CTA) or 256 (CTA pair), tile_n 64 / 128 / 256, stages 0 = deepest ring that fits, splitK >= 1 (0 = the
// library's rule), streamK 0 / 1, kpr = K blocks per barrier round (1 / 2 / 4; absent or 0 = the library's rule).
// The reference's own strings - "v2:M,N,KpackPerBlock,MPerWave,NPerWave,KPack,SplitK,ForceUnroll,ThreadCopyMore" and
// the un-prefixed version 1 (mlir/include/mlir/Dialect/Rock/Tuning/GridwiseGemmParams.h:138-194,
// Serializable.h:37-131) - are accepted too and mapped onto the nearest tile with the K split honoured.
bool perf_config_to_variant(const char* str, uint32_t* variant);
std::string variant_to_perf_config(uint32_t variant);

}  // namespace rb
