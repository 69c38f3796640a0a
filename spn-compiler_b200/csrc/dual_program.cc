// Host-side planning for the two-tile tcgen05 layered kernel (layered_tcf_dual.cu): annotates the post-order
// region program with where every region's outputs go (a-stack slot, MMA operand buffer, registers, root) and
// lists the leaf stages (four features each) in execution order.
#include <algorithm>
#include <sstream>

#include "layered.h"
#include "layers.h"

namespace spnb {

bool buildDualProgram(const LayeredPlan& lp, const std::vector<long long>& fragOffset, const std::vector<int>& blocks,
                      const std::vector<int>& scaleOffset, const std::vector<float>& centres, DualProgram* out) {
  *out = DualProgram();
  const size_t ns = lp.steps.size();
  std::vector<int> consumer(ns, -1), side(ns, 0);   // side: 0 left operand, 1 right operand
  std::vector<int> stack;
  for (size_t i = 0; i < ns; ++i) {
    const LayerStep& s = lp.steps[i];
    if (s.op == kLeafRegion) {
      if (s.width > 32) return false;
      stack.push_back((int)i);
      continue;
    }
    // every inner region must have tensor-core weights (32 x 32 cross products, at most 32 sums), and its right
    // operand must be the step directly before it (true for every post-order walk of a binary region tree)
    if (stack.size() < 2 || fragOffset[i] < 0) return false;
    const int b = stack.back();
    stack.pop_back();
    const int a = stack.back();
    stack.pop_back();
    if (b != (int)i - 1) return false;
    consumer[(size_t)a] = (int)i;
    side[(size_t)a] = 0;
    consumer[(size_t)b] = (int)i;
    side[(size_t)b] = 1;
    if (s.op == kInnerRegion) stack.push_back((int)i);
  }
  if (!stack.empty()) return false;

  out->steps.resize(ns);
  int depth = 0;
  for (size_t i = 0; i < ns; ++i) {
    const LayerStep& s = lp.steps[i];
    DualStepDev& d = out->steps[i];
    d = DualStepDev{};
    d.op = s.op;
    d.width = s.width;
    d.aSrc = -1;
    if (s.op == kLeafRegion) {
      d.numFeatures = s.numFeatures;
      d.featOffset = (int)s.featOffset;
      d.paramOffset = (long long)s.paramOffset;
      if (fragOffset[i] >= 0) {
        const int nst = (s.numFeatures + 7) / 8;
        d.numBlocks = nst;
        d.fragOffset = fragOffset[i] * 8;
        d.stageBase = (int)(out->cols4.size() / 8);
        for (int q = 0; q < nst * 8; ++q) {
          out->cols4.push_back(q < s.numFeatures ? lp.features[(size_t)s.featOffset + q] : 0);
          out->centres4.push_back(q < s.numFeatures ? centres[(size_t)s.featOffset + q] : 0.f);
        }
      }
    } else {
      // the left operand is popped from the a-stack unless its producer kept it in registers (the producer is
      // two steps back and the step in between is the single leaf region that makes the right operand)
      const bool aInRegs = i >= 2 && lp.steps[i - 1].op == kLeafRegion && consumer[i - 2] == (int)i;
      if (!aInRegs) {
        if (depth == 0) return false;
        d.aSrc = --depth;
      }
      d.numBlocks = blocks[i];
      d.fragOffset = fragOffset[i] * 8;
      d.scaleOffset = scaleOffset[i];
    }
    if (s.op == kRootPart) d.dest = kDualDestRoot;
    else if (side[i] == 1) d.dest = kDualDestOperand;
    else if (consumer[i] == (int)i + 2 && lp.steps[i + 1].op == kLeafRegion) d.dest = kDualDestRegs;
    else {
      d.dest = kDualDestStack;
      d.destSlot = depth++;
      out->aSlots = std::max(out->aSlots, depth);
    }
  }
  if (depth != 0) return false;
  out->aSlots = std::max(out->aSlots, 1);
  return true;
}

std::string dualProgramSummary(const DualProgram& p) {
  // one letter per step: leaf / inner / root part in upper case, followed by the destination (s<slot>, o, r, -)
  // and, for inner steps, the source of the left operand (<slot> or r)
  std::ostringstream o;
  o << "{\"a_slots\":" << p.aSlots << ",\"leaf_stages\":" << p.cols4.size() / 8 << ",\"steps\":\"";
  for (const DualStepDev& d : p.steps) {
    o << (d.op == kLeafRegion ? 'L' : (d.op == kInnerRegion ? 'I' : 'R'));
    if (d.op != kLeafRegion) {
      if (d.aSrc >= 0) o << d.aSrc;
      else o << 'r';
    }
    switch (d.dest) {
      case kDualDestStack: o << 's' << d.destSlot; break;
      case kDualDestOperand: o << 'o'; break;
      case kDualDestRegs: o << 'r'; break;
      default: o << '-';
    }
    o << ' ';
  }
  o << "\"}";
  return o.str();
}

}  // namespace spnb
