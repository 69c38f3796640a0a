// Recognition of layered (RAT-SPN-style) structure in a canonical DAG and the flat description the
// layered kernel executes.  The xspn format has no notion of layers: a RAT-SPN arrives as hundreds of
// thousands of nodes and millions of sum edges, and is re-assembled here into regions.
#pragma once
#include <cstdint>
#include <vector>

#include "plan.h"

namespace spnb {

// One step of the layered program (a stack machine over region outputs, post-order over the region tree).
//   kLeafRegion:  push `width` values:  out_k = sum_f c2_kf * (x_f - mu_kf)^2 + c1_kf
//   kInnerRegion: pop b (top, width wb), pop a (width wa), push `width` values:
//                 out_k = max(a) + max(b) + log2( sum_ij W_k[i*wb+j] * 2^(a_i - max a) * 2^(b_j - max b) )
//   kRootPart:    like kInnerRegion with one output, which is folded into the running root log-sum
enum LayerOp : int32_t { kLeafRegion = 0, kInnerRegion = 1, kRootPart = 2 };

struct LayerStep {
  int32_t op = 0;
  int32_t width = 0;          // outputs
  int32_t wa = 0, wb = 0;     // widths of the two operands (inner / root part)
  int32_t numFeatures = 0;    // leaf region
  int64_t featOffset = 0;     // leaf: first entry in LayeredPlan::features
  int64_t paramOffset = 0;    // leaf: first 4-float entry in leafParams (layout [feature][k]); inner: first float in weights
};

struct LayeredPlan {
  std::vector<LayerStep> steps;
  std::vector<int32_t> features;   // input columns of the leaf regions
  std::vector<float> leafParams;   // (mu, c2, c1, 0) of the Gaussian log2-density c2*(x - mu)^2 + c1: the centred form the
                                   // reference evaluates (an expanded quadratic cancels badly when |mu| >> stddev)
  std::vector<float> weights;      // linear-space sum weights, [k][i*wb + j]
  int32_t maxWidth = 0;
  int32_t maxDepth = 0;            // deepest the region stack gets
  int32_t maxLeafFeatures = 0;
};

// True if the whole DAG is a root sum over cross products of region outputs, regions being either groups
// of sums sharing one ordered list of cross products of two regions, or groups of products of Gaussian
// leaves over one feature set.  Fills `out` on success.
bool recogniseLayers(const Dag& d, LayeredPlan* out);

}  // namespace spnb
