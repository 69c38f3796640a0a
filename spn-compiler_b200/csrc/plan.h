// Planner: turns a validated Model into an evaluation-ordered, de-duplicated DAG plus the
// device-side tables and (for the interpreter kernel) an op stream with liveness-based slots.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "model.h"

namespace spnb {

// Canonical DAG: only nodes reachable from the root, structurally identical nodes merged
// (what the reference obtains from CSE + canonicalisation,
// compiler/src/pipeline/steps/mlir/transformation/LoSPNTransformations.cpp:21-23), single-operand
// products folded away, numbered in evaluation order (children before parents, root last).
struct Dag {
  int32_t numFeatures = 0;
  std::vector<uint8_t> kind;
  std::vector<int32_t> feature;
  std::vector<double> mean, stddev;
  std::vector<int64_t> childPtr;
  std::vector<int32_t> childIdx;
  std::vector<double> weight;
  std::vector<int64_t> tabPtr;
  std::vector<double> tab;
  std::vector<int64_t> brkPtr;
  std::vector<int32_t> brk;
  std::vector<int32_t> uses;   // number of parents edges per node
  std::vector<int32_t> group;  // discrete leaves: index group; -1 otherwise
  int32_t root() const { return (int32_t)kind.size() - 1; }
  size_t size() const { return kind.size(); }
};

// Discrete inputs are digested once per (sample, feature) while the input tile is staged:
//   code = 0 for NaN, 1 outside [lo, lo + domain), else 2 + (trunc(x) - lo)
// where [lo, lo + domain) covers every bucket / category of every discrete leaf on the feature.
// A feature read by Gaussian leaves is (also) staged as a real value.
struct FeatureMeta {
  int32_t lo = 0;
  int32_t domain = 0;
  int32_t codeSlot = -1;   // row of the staged code array, -1: no discrete leaf reads the feature
  int32_t valueSlot = -1;  // row of the staged value array, -1: no leaf needs the value itself
  // every discrete leaf on the feature buckets its input arithmetically (IndexGroup::clampFit): a generated
  // kernel may stage missing inputs as code 65535 and out-of-range ones as domain + 2 instead of 0 and 1
  bool clampCodes = false;
};

// All discrete leaves on one feature that bucket the input the same way form a group.
enum GroupMode : int32_t {
  kDirect = 0,   // leaf table indexed by the code itself (domain + 2 entries): categorical, narrow histograms
  kLut = 1,      // byte table code -> bucket, then a (buckets + 2)-entry leaf table
  kGeneric = 2,  // domain too wide for a byte table: compare against the breaks
};
struct IndexGroup {
  int32_t feature = 0;
  bool histogram = false;
  int32_t count = 0;             // categories K, or number of buckets
  std::vector<int32_t> breaks;   // histogram only: count+1 ascending bounds
  int32_t mode = kDirect;
  int32_t lutOffset = -1;        // kLut: first entry in Plan::lut (identical tables are shared)
  int32_t brkOffset = -1;        // kGeneric: first break in Plan::groupBreaks
  // kLut groups whose byte table is reproduced exactly by  bucket = (code * arMul + arAdd) >> 16  for every
  // code >= 2 (near-equal-width buckets): generated kernels may compute the bucket instead of loading it
  bool arith = false;
  int32_t arMul = 0, arAdd = 0;
  // ... and a second fit that also sends the code one past the domain (domain + 2) to bucket `count`, the
  // out-of-range entry, and the largest 16-bit code to at least count + 1: with the feature's missing inputs
  // staged as 65535 and its out-of-range inputs as domain + 2 (FeatureMeta::clampCodes), the table index is
  // min((code * clMul + clAdd) >> 16, count + 1) with no special cases and no byte table
  bool clampFit = false;
  int32_t clMul = 0, clAdd = 0;
};

struct PlanStats {
  int64_t nodes = 0, sums = 0, products = 0, gauss = 0, cats = 0, hists = 0;
  int64_t sumEdges = 0, productEdges = 0;
  int64_t depth = 0;
  int64_t modelNodes = 0;     // nodes in the file
  // algorithmic work per sample (log-space f32 formulation: n-ary max-shifted log-sum-exp)
  int64_t opsSfu = 0;         // sum over sums of (k + 1): k exp2 + 1 log2
  int64_t opsFp32 = 0;        // 3/gauss + 2/discrete leaf + (k-1)/product + (4k-1)/sum + opsSfu
  int64_t opsFp64 = 0;        // linear f64 formulation: (k-1)/product + (2k-1)/sum + leaves + 40 (root log)
  int64_t bytesPerSample = 0; // F * sizeof(input) + sizeof(output)
  // The reference's graph statistics (mlir/lib/Dialect/LoSPN/Passes/LoSPNGraphStatsCollection.cpp:83-102),
  // counted on the form the reference lowers to: a product / weighted sum with k operands is a balanced tree
  // of k-1 two-input multiplications / additions, every sum operand is first multiplied by a weight constant
  // (equal constants are one node after CSE).  Depths are the levels of the distinct leaves below the root
  // (root = level 0) in that two-input form.
  int64_t featureCount = 0, refAdds = 0, refMuls = 0, refConstants = 0;
  int64_t minDepth = 0, maxDepth = 0;
  double averageDepth = 0.0, medianDepth = 0.0;
  std::string toJson() const;
  // JSON object with exactly the reference's keys: featureCount, minDepth, maxDepth, averageDepth, medianDepth,
  // innerCount, leafCount, sumCount, productCount, categoricalCount, constantCount, gaussianCount, histogramCount
  std::string toReferenceJson() const;
};

// Interpreter program: a flat int32 stream, all operands are value slots.
//   OP_GAUSS  dst f  mu c2 c1            (floats bit-cast; linear space: indices of mean, exponent factor, coefficient)
//   OP_TABLE  dst codeSlot lutOffset(-1: direct) tabOffset
//   OP_HISTG  dst valueSlot brkOffset count tabOffset      (generic histogram)
//   OP_PROD   dst k  s_0 .. s_{k-1}
//   OP_SUM    dst k  (s_i w_i) * k        (w_i = log2 weight, bit-cast; linear space: index of the weight)
//   OP_END    src
enum InterpOp : int32_t { OP_END = 0, OP_GAUSS = 1, OP_TABLE = 2, OP_PROD = 3, OP_SUM = 4, OP_HISTG = 5 };

struct Plan {
  bool logSpace = true;       // false: linear f64 with one root log (the reference's f64 mode)
  bool marginal = false;
  FeatureType ftype;
  Dag dag;
  std::vector<IndexGroup> groups;
  std::vector<FeatureMeta> features;
  int32_t numCodeSlots = 0, numValueSlots = 0;
  std::vector<uint8_t> lut;         // byte tables of the kLut groups
  // leaf tables.  kDirect: [0] NaN input, [1] out of range, [2 + i] value of lo + i.
  // kLut / kGeneric: [0 .. count) bucket values, [count] out of range, [count + 1] NaN input.
  std::vector<int32_t> tabOffset;   // per node, -1 if none
  std::vector<float> tabF32;        // log2 domain
  std::vector<double> tabF64;       // probabilities
  PlanStats stats;
  // interpreter
  std::vector<int32_t> prog;
  // linear-space programs name their constants by index into this table: OP_GAUSS carries (mean, -1/(2 var),
  // 1/sqrt(2 pi var)) as three indices, OP_SUM one index per weight
  std::vector<double> progConsts;
  std::vector<int32_t> groupBreaks; // breaks of the kGeneric groups
  int32_t numSlots = 0;       // slots needed when every value lives in shared memory
  int32_t numSmemSlots = 0;   // of the current program: shared-memory slots ...
  int32_t numSpillSlots = 0;  // ... and slots in global scratch memory (ids numSmemSlots' capacity and up)
};

Dag canonicalize(const Model& m);
Plan buildPlan(const Model& m, bool logSpace);
// (Re)builds Plan::prog with at most smemSlots values in shared memory (INT32_MAX: no limit).
void buildProgram(Plan& p, int32_t smemSlots);

}  // namespace spnb
