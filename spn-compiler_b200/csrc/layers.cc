#include "layers.h"

#include <algorithm>
#include <cmath>
#include <functional>
#include <map>

namespace spnb {

namespace {

struct Recogniser {
  const Dag& d;
  LayeredPlan& lp;
  std::map<int32_t, int32_t> depthMemo;
  explicit Recogniser(const Dag& dag, LayeredPlan& out) : d(dag), lp(out) {}

  int64_t nkids(int32_t v) const { return d.childPtr[v + 1] - d.childPtr[v]; }
  int32_t kid(int32_t v, int64_t i) const { return d.childIdx[d.childPtr[v] + i]; }

  // Splits a list of two-operand products starting at `pos` into one cross-product block a x b.
  // Returns the number of products consumed (wa * wb) or 0 if the structure does not match.
  int64_t crossBlock(const int32_t* list, int64_t count, int64_t pos, std::vector<int32_t>* a, std::vector<int32_t>* b) const {
    a->clear();
    b->clear();
    auto isPair = [&](int32_t v) { return d.kind[v] == kProduct && nkids(v) == 2; };
    if (pos >= count || !isPair(list[pos])) return 0;
    const int32_t a0 = kid(list[pos], 0);
    int64_t wb = 0;
    while (pos + wb < count && isPair(list[pos + wb]) && kid(list[pos + wb], 0) == a0) {
      b->push_back(kid(list[pos + wb], 1));
      ++wb;
    }
    if (std::find(b->begin() + 1, b->end(), (*b)[0]) != b->end()) return 0;
    int64_t wa = 0;
    for (;;) {
      const int64_t base = pos + wa * wb;
      if (base + wb > count || !isPair(list[base])) break;
      const int32_t ai = kid(list[base], 0);
      if (wa > 0 && std::find(a->begin(), a->end(), ai) != a->end()) break;
      bool ok = true;
      for (int64_t j = 0; j < wb && ok; ++j)
        ok = isPair(list[base + j]) && kid(list[base + j], 0) == ai && kid(list[base + j], 1) == (*b)[j];
      if (!ok) break;
      a->push_back(ai);
      ++wa;
    }
    return wa ? wa * wb : 0;
  }

  // Emits the steps that leave the values of `nodes` (one region) on top of the stack.
  // Returns the stack depth needed, or -1 on mismatch.
  int region(const std::vector<int32_t>& nodes) {
    if (nodes.empty()) return -1;
    const int32_t first = nodes[0];
    if (d.kind[first] == kProduct) {
      // leaf region: every node is a product of Gaussian leaves over one and the same feature list
      const int64_t nf = nkids(first);
      std::vector<int32_t> feats;
      for (int64_t f = 0; f < nf; ++f) {
        if (d.kind[kid(first, f)] != kGaussian) return -1;
        feats.push_back(d.feature[kid(first, f)]);
      }
      LayerStep s;
      s.op = kLeafRegion;
      s.width = (int32_t)nodes.size();
      s.numFeatures = (int32_t)nf;
      s.featOffset = (int64_t)lp.features.size();
      s.paramOffset = (int64_t)lp.leafParams.size() / 4;
      lp.features.insert(lp.features.end(), feats.begin(), feats.end());
      lp.leafParams.resize(lp.leafParams.size() + 4 * (size_t)nf * nodes.size(), 0.f);
      const double LOG2E = 1.4426950408889634074;
      for (size_t k = 0; k < nodes.size(); ++k) {
        const int32_t v = nodes[k];
        if (d.kind[v] != kProduct || nkids(v) != nf) return -1;
        for (int64_t f = 0; f < nf; ++f) {
          const int32_t g = kid(v, f);
          if (d.kind[g] != kGaussian || d.feature[g] != feats[(size_t)f]) return -1;
          const double sd = d.stddev[g], mu = d.mean[g];
          const double c2 = -(1.0 / (2.0 * sd * sd)) * LOG2E;
          const double c1 = (-std::log(sd) - 0.5 * std::log(2 * M_PI)) * LOG2E;
          const size_t q = 4 * ((size_t)s.paramOffset + (size_t)f * nodes.size() + k);
          lp.leafParams[q] = (float)mu;
          lp.leafParams[q + 1] = (float)c2;
          lp.leafParams[q + 2] = (float)c1;
        }
      }
      lp.maxWidth = std::max(lp.maxWidth, s.width);
      lp.maxLeafFeatures = std::max(lp.maxLeafFeatures, s.numFeatures);
      lp.steps.push_back(s);
      return 1;
    }
    if (d.kind[first] != kSum) return -1;
    // inner region: sums over one shared ordered list of cross products
    const int64_t n = nkids(first);
    const int32_t* list = &d.childIdx[d.childPtr[first]];
    for (int32_t v : nodes) {
      if (d.kind[v] != kSum || nkids(v) != n) return -1;
      if (!std::equal(list, list + n, &d.childIdx[d.childPtr[v]])) return -1;
    }
    std::vector<int32_t> a, b;
    if (crossBlock(list, n, 0, &a, &b) != n) return -1;
    const int da = region(a);
    if (da < 0) return -1;
    const int db = region(b);
    if (db < 0) return -1;
    LayerStep s;
    s.op = kInnerRegion;
    s.width = (int32_t)nodes.size();
    s.wa = (int32_t)a.size();
    s.wb = (int32_t)b.size();
    s.paramOffset = (int64_t)lp.weights.size();
    for (int32_t v : nodes)
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) lp.weights.push_back((float)d.weight[e]);
    lp.maxWidth = std::max({lp.maxWidth, s.width, s.wa, s.wb});
    lp.steps.push_back(s);
    return std::max(da, 1 + db);
  }
};

}  // namespace

bool recogniseLayers(const Dag& d, LayeredPlan* out) {
  *out = LayeredPlan();
  const int32_t root = d.root();
  if (d.kind[root] != kSum) return false;
  Recogniser r(d, *out);
  const int64_t n = r.nkids(root);
  if (n < 4) return false;
  const int32_t* list = &d.childIdx[d.childPtr[root]];
  std::vector<int32_t> a, b;
  int64_t pos = 0;
  int depth = 0;
  while (pos < n) {
    const int64_t used = r.crossBlock(list, n, pos, &a, &b);
    if (!used || a.size() < 2 || b.size() < 2) return false;
    const int da = r.region(a);
    if (da < 0) return false;
    const int db = r.region(b);
    if (db < 0) return false;
    LayerStep s;
    s.op = kRootPart;
    s.width = 1;
    s.wa = (int32_t)a.size();
    s.wb = (int32_t)b.size();
    s.paramOffset = (int64_t)out->weights.size();
    for (int64_t e = 0; e < used; ++e) out->weights.push_back((float)d.weight[d.childPtr[root] + pos + e]);
    out->steps.push_back(s);
    depth = std::max({depth, da, 1 + db});
    pos += used;
  }
  out->maxDepth = depth;
  // the kernel keeps one operand per register: widths are bounded
  if (out->maxWidth > 32 || out->maxWidth < 1) return false;
  return true;
}

}  // namespace spnb
