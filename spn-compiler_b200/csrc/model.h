// In-memory form of an xspn model/query and the validation rules of the front end.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace spnb {

// Union order of `Node` in the xspn schema (spflow.capnp:56-67 of the reference).
enum NodeKind : uint8_t { kProduct = 0, kSum = 1, kHistogram = 2, kGaussian = 3, kCategorical = 4 };

enum class InKind : uint8_t { Int, UInt, Float };

struct FeatureType {
  InKind kind = InKind::Float;
  int bits = 64;
  int bytes() const { return bits >> 3; }
  bool isFloat() const { return kind == InKind::Float; }
};

// Parses a numpy dtype name the way the reference's front end does
// (compiler/src/pipeline/steps/frontend/SPFlowToMLIRDeserializer.cpp:226-248): "[u]int<W>" or
// "float<W>" with W in {16,32,64} for floats.  Throws on anything else.
FeatureType parseFeatureType(const std::string& text);

struct Model {
  bool isQuery = false;
  int32_t batchSize = 1;
  int32_t errorKind = 0;  // 0 absolute, 1 relative
  double maxError = 0.0;
  bool supportMarginal = false;

  std::string name;         // empty name becomes "spn_kernel"
  std::string featureType;  // numpy dtype name
  FeatureType ftype;
  int32_t numFeatures = 0;  // = size of the model's scope

  // Nodes in file order (children before parents); struct-of-arrays.
  std::vector<uint8_t> kind;
  std::vector<int32_t> feature;  // input column of a leaf (position of its feature id in the sorted scope)
  std::vector<double> mean, stddev;
  std::vector<int64_t> childPtr;   // n+1
  std::vector<int32_t> childIdx;   // node indices
  std::vector<double> weight;      // aligned with childIdx; 0 for product edges
  std::vector<int64_t> tabPtr;     // n+1: categorical probabilities / histogram densities
  std::vector<double> tab;
  std::vector<int64_t> brkPtr;     // n+1: histogram breaks
  std::vector<int32_t> brk;
  int32_t root = -1;

  size_t numNodes() const { return kind.size(); }
};

// Throws std::runtime_error with the reference's wording when a rule of its verifiers is broken
// (mlir/lib/Dialect/HiSPN/HiSPNOps.cpp:33-126): marginal support needs a floating feature type,
// products/sums need operands, #weights == #addends, |sum(w) - 1| <= 1e-6, categorical
// probabilities sum to 1 +- 1e-6, histogram buckets ordered and non-overlapping.
void validateModel(const Model& m);

// Reads an xspn file (Cap'n Proto, unpacked stream framing, any number of segments).
// Accepts both header kinds: a query (the only one the reference compiles) and a bare model
// (batchSize 1, no marginal support), so that the stored example models are usable directly.
Model readXspnFile(const std::string& path);
Model readXspnBytes(const uint8_t* data, size_t size);

}  // namespace spnb
