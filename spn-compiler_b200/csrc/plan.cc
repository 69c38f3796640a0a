#include "plan.h"

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstring>
#include <map>
#include <sstream>
#include <unordered_map>

namespace spnb {

namespace {

struct Key128 {
  uint64_t a, b;
  bool operator==(const Key128& o) const { return a == o.a && b == o.b; }
};
struct KeyHash {
  size_t operator()(const Key128& k) const { return (size_t)(k.a ^ (k.b * 0x9E3779B97F4A7C15ull)); }
};

struct Hasher {
  uint64_t a = 0xcbf29ce484222325ull, b = 0x84222325cbf29ce4ull;
  void add(uint64_t v) {
    a = (a ^ v) * 0x100000001b3ull;
    a ^= a >> 29;
    b = (b + v) * 0xff51afd7ed558ccdull;
    b ^= b >> 32;
  }
  void addDouble(double d) {
    uint64_t u;
    std::memcpy(&u, &d, 8);
    add(u);
  }
  Key128 key() const { return Key128{a, b}; }
};

inline uint32_t f32bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}

}  // namespace

Dag canonicalize(const Model& m) {
  const size_t n = m.numNodes();
  // ---- phase A: hash-consing in file order ------------------------------------------------
  std::vector<int32_t> canon(n, -1);
  std::vector<int32_t> uNode;  // unique id -> a representative model node
  std::vector<int64_t> uChildPtr{0};
  std::vector<int32_t> uChild;
  std::unordered_multimap<Key128, int32_t, KeyHash> seen;
  seen.reserve(n * 2);
  // structural equality of model node v with the representative of unique node u (the hash only nominates)
  auto sameNode = [&](size_t v, int32_t u) {
    const int32_t r = uNode[(size_t)u];
    if (m.kind[v] != m.kind[r]) return false;
    const int64_t lo = m.childPtr[v], hi = m.childPtr[v + 1], rlo = m.childPtr[r];
    if (hi - lo != m.childPtr[r + 1] - rlo) return false;
    if (m.kind[v] == kProduct || m.kind[v] == kSum) {
      for (int64_t e = 0; e < hi - lo; ++e) {
        if (canon[m.childIdx[lo + e]] != uChild[(size_t)(uChildPtr[(size_t)u] + e)]) return false;
        if (m.kind[v] == kSum && m.weight[lo + e] != m.weight[rlo + e]) return false;
      }
      return true;
    }
    if (m.feature[v] != m.feature[r]) return false;
    if (m.kind[v] == kGaussian) return m.mean[v] == m.mean[r] && m.stddev[v] == m.stddev[r];
    const int64_t nt = m.tabPtr[v + 1] - m.tabPtr[v], nb = m.brkPtr[v + 1] - m.brkPtr[v];
    if (nt != m.tabPtr[r + 1] - m.tabPtr[r] || nb != m.brkPtr[r + 1] - m.brkPtr[r]) return false;
    return std::equal(m.tab.begin() + m.tabPtr[v], m.tab.begin() + m.tabPtr[v + 1], m.tab.begin() + m.tabPtr[r]) &&
           std::equal(m.brk.begin() + m.brkPtr[v], m.brk.begin() + m.brkPtr[v + 1], m.brk.begin() + m.brkPtr[r]);
  };
  for (size_t v = 0; v < n; ++v) {
    int64_t lo = m.childPtr[v], hi = m.childPtr[v + 1];
    uint8_t kind = m.kind[v];
    if (kind == kProduct && hi - lo == 1) {
      canon[v] = canon[m.childIdx[lo]];
      continue;
    }
    Hasher h;
    h.add(kind);
    h.add((uint64_t)(hi - lo));
    if (kind == kProduct || kind == kSum) {
      for (int64_t e = lo; e < hi; ++e) {
        h.add((uint64_t)(uint32_t)canon[m.childIdx[e]]);
        if (kind == kSum) h.addDouble(m.weight[e]);
      }
    } else {
      h.add((uint64_t)(uint32_t)m.feature[v]);
      if (kind == kGaussian) {
        h.addDouble(m.mean[v]);
        h.addDouble(m.stddev[v]);
      } else {
        h.add((uint64_t)(m.tabPtr[v + 1] - m.tabPtr[v]));
        for (int64_t t = m.tabPtr[v]; t < m.tabPtr[v + 1]; ++t) h.addDouble(m.tab[t]);
        for (int64_t t = m.brkPtr[v]; t < m.brkPtr[v + 1]; ++t) h.add((uint64_t)(uint32_t)m.brk[t]);
      }
    }
    const Key128 key = h.key();
    int32_t found = -1;
    auto range = seen.equal_range(key);
    for (auto it = range.first; it != range.second && found < 0; ++it)
      if (sameNode(v, it->second)) found = it->second;
    if (found >= 0) {
      canon[v] = found;
      continue;
    }
    seen.emplace(key, (int32_t)uNode.size());
    canon[v] = (int32_t)uNode.size();
    uNode.push_back((int32_t)v);
    for (int64_t e = lo; e < hi; ++e) uChild.push_back(canon[m.childIdx[e]]);
    uChildPtr.push_back((int64_t)uChild.size());
  }
  const size_t nu = uNode.size();
  // ---- phase B: evaluation order = DFS post-order, register-hungry subtrees first ----------
  std::vector<int32_t> need(nu, 1);
  std::vector<int32_t> tmp;
  for (size_t u = 0; u < nu; ++u) {
    int64_t lo = uChildPtr[u], hi = uChildPtr[u + 1];
    if (hi == lo) continue;
    tmp.assign(uChild.begin() + lo, uChild.begin() + hi);
    std::sort(tmp.begin(), tmp.end(), [&](int32_t x, int32_t y) { return need[x] > need[y]; });
    int32_t best = 1;
    for (size_t i = 0; i < tmp.size(); ++i) best = std::max(best, need[tmp[i]] + (int32_t)i);
    need[u] = best;
  }
  std::vector<int32_t> newId(nu, -1);
  std::vector<int32_t> order;
  order.reserve(nu);
  {
    struct Frame { int32_t u; int32_t next; };
    std::vector<Frame> stack;
    std::vector<std::vector<int32_t>> visit;  // per stack depth: children in visiting order
    stack.push_back({canon[m.root], 0});
    std::vector<uint8_t> state(nu, 0);  // 0 new, 1 open, 2 done
    std::vector<int32_t> sortedKids;
    std::vector<int64_t> kidsPtr(nu + 1, 0);
    // visiting order per node, computed lazily into a side CSR
    std::vector<int32_t> vo;
    std::vector<int64_t> voStart(nu, -1);
    while (!stack.empty()) {
      Frame& f = stack.back();
      int32_t u = f.u;
      if (state[u] == 2) { stack.pop_back(); continue; }
      if (state[u] == 0) {
        state[u] = 1;
        int64_t lo = uChildPtr[u], hi = uChildPtr[u + 1];
        voStart[u] = (int64_t)vo.size();
        vo.insert(vo.end(), uChild.begin() + lo, uChild.begin() + hi);
        std::stable_sort(vo.begin() + voStart[u], vo.end(), [&](int32_t x, int32_t y) { return need[x] > need[y]; });
      }
      int64_t cnt = uChildPtr[u + 1] - uChildPtr[u];
      bool pushed = false;
      while (f.next < cnt) {
        int32_t c = vo[voStart[u] + f.next];
        f.next++;
        if (state[c] == 0) {
          stack.push_back({c, 0});
          pushed = true;
          break;
        }
      }
      if (pushed) continue;
      state[u] = 2;
      newId[u] = (int32_t)order.size();
      order.push_back(u);
      stack.pop_back();
    }
    (void)sortedKids; (void)kidsPtr; (void)visit;
  }
  // ---- build the Dag ----------------------------------------------------------------------
  Dag d;
  d.numFeatures = m.numFeatures;
  const size_t nd = order.size();
  d.kind.resize(nd);
  d.feature.assign(nd, -1);
  d.mean.assign(nd, 0.0);
  d.stddev.assign(nd, 1.0);
  d.childPtr.assign(nd + 1, 0);
  d.tabPtr.assign(nd + 1, 0);
  d.brkPtr.assign(nd + 1, 0);
  d.uses.assign(nd, 0);
  d.group.assign(nd, -1);
  for (size_t i = 0; i < nd; ++i) {
    int32_t u = order[i];
    int32_t v = uNode[u];
    d.kind[i] = m.kind[v];
    d.feature[i] = m.feature[v];
    d.mean[i] = m.mean[v];
    d.stddev[i] = m.stddev[v];
    for (int64_t e = m.childPtr[v]; e < m.childPtr[v + 1]; ++e) {
      int32_t c = newId[canon[m.childIdx[e]]];
      d.childIdx.push_back(c);
      d.weight.push_back(m.weight[e]);
      d.uses[c]++;
    }
    d.tab.insert(d.tab.end(), m.tab.begin() + m.tabPtr[v], m.tab.begin() + m.tabPtr[v + 1]);
    d.brk.insert(d.brk.end(), m.brk.begin() + m.brkPtr[v], m.brk.begin() + m.brkPtr[v + 1]);
    d.childPtr[i + 1] = (int64_t)d.childIdx.size();
    d.tabPtr[i + 1] = (int64_t)d.tab.size();
    d.brkPtr[i + 1] = (int64_t)d.brk.size();
  }
  return d;
}

std::string PlanStats::toJson() const {
  std::ostringstream o;
  o << "{\"model_nodes\":" << modelNodes << ",\"nodes\":" << nodes << ",\"sums\":" << sums << ",\"products\":" << products
    << ",\"gaussian\":" << gauss << ",\"categorical\":" << cats << ",\"histogram\":" << hists
    << ",\"sum_edges\":" << sumEdges << ",\"product_edges\":" << productEdges << ",\"depth\":" << depth
    << ",\"ops_sfu\":" << opsSfu << ",\"ops_fp32\":" << opsFp32 << ",\"ops_fp64\":" << opsFp64
    << ",\"bytes_per_sample\":" << bytesPerSample << "}";
  return o.str();
}

std::string PlanStats::toReferenceJson() const {
  std::ostringstream o;
  o << "{\"featureCount\":" << featureCount << ",\"minDepth\":" << minDepth << ",\"maxDepth\":" << maxDepth
    << ",\"averageDepth\":" << averageDepth << ",\"medianDepth\":" << medianDepth
    << ",\"innerCount\":" << (refAdds + refMuls) << ",\"leafCount\":" << (gauss + cats + hists + refConstants)
    << ",\"sumCount\":" << refAdds << ",\"productCount\":" << refMuls << ",\"categoricalCount\":" << cats
    << ",\"constantCount\":" << refConstants << ",\"gaussianCount\":" << gauss << ",\"histogramCount\":" << hists << "}";
  return o.str();
}

Plan buildPlan(const Model& m, bool logSpace) {
  Plan p;
  p.logSpace = logSpace;
  p.marginal = m.supportMarginal;
  p.ftype = m.ftype;
  p.dag = canonicalize(m);
  Dag& d = p.dag;
  const size_t n = d.size();

  // ---- index groups, staged-feature layout and leaf tables --------------------------------------
  const int32_t F = d.numFeatures;
  p.features.assign(F, FeatureMeta{});
  std::vector<int64_t> flo(F, INT64_MAX), fhi(F, INT64_MIN);
  std::map<std::vector<int32_t>, int32_t> groupOf;
  p.tabOffset.assign(n, -1);
  std::vector<int32_t> key;
  for (size_t v = 0; v < n; ++v) {
    if (d.kind[v] == kGaussian) {
      FeatureMeta& fm = p.features[d.feature[v]];
      if (fm.valueSlot < 0) fm.valueSlot = p.numValueSlots++;
      continue;
    }
    if (d.kind[v] != kCategorical && d.kind[v] != kHistogram) continue;
    bool hist = d.kind[v] == kHistogram;
    int32_t count = (int32_t)(d.tabPtr[v + 1] - d.tabPtr[v]);
    key.clear();
    key.push_back(d.feature[v]);
    key.push_back(hist ? 1 : 0);
    key.push_back(count);
    if (hist) key.insert(key.end(), d.brk.begin() + d.brkPtr[v], d.brk.begin() + d.brkPtr[v + 1]);
    auto ins = groupOf.emplace(key, (int32_t)p.groups.size());
    if (ins.second) {
      IndexGroup g;
      g.feature = d.feature[v];
      g.histogram = hist;
      g.count = count;
      if (hist) g.breaks.assign(d.brk.begin() + d.brkPtr[v], d.brk.begin() + d.brkPtr[v + 1]);
      int64_t lo = hist ? g.breaks.front() : 0, hi = hist ? g.breaks.back() : count;
      flo[g.feature] = std::min(flo[g.feature], lo);
      fhi[g.feature] = std::max(fhi[g.feature], hi);
      p.groups.push_back(std::move(g));
    }
    d.group[v] = ins.first->second;
  }
  const int64_t kMaxDomain = 65000;
  for (int32_t f = 0; f < F; ++f) {
    if (flo[f] > fhi[f]) continue;
    FeatureMeta& fm = p.features[f];
    if (fhi[f] - flo[f] <= kMaxDomain) {
      fm.lo = (int32_t)flo[f];
      fm.domain = (int32_t)(fhi[f] - flo[f]);
      fm.codeSlot = p.numCodeSlots++;
    }
  }
  std::map<std::vector<uint8_t>, int32_t> lutOf;
  for (IndexGroup& g : p.groups) {
    FeatureMeta& fm = p.features[g.feature];
    const int64_t entries = (int64_t)fm.domain + 2;
    if (fm.codeSlot < 0 || (g.histogram && g.count + 2 > 255 && entries > 2 * ((int64_t)g.count + 2))) {
      if (!g.histogram) throw std::runtime_error("Categorical leaf with too many categories");
      g.mode = kGeneric;
      g.brkOffset = (int32_t)p.groupBreaks.size();
      p.groupBreaks.insert(p.groupBreaks.end(), g.breaks.begin(), g.breaks.end());
      if (fm.valueSlot < 0) fm.valueSlot = p.numValueSlots++;
    } else if (!g.histogram || entries <= 2 * ((int64_t)g.count + 2)) {
      g.mode = kDirect;
    } else {
      g.mode = kLut;
      std::vector<uint8_t> lut((size_t)entries);
      lut[0] = (uint8_t)(g.count + 1);
      lut[1] = (uint8_t)g.count;
      int32_t b = 0;
      for (int32_t i = 0; i < fm.domain; ++i) {
        int64_t x = (int64_t)fm.lo + i;
        while (b < g.count && x >= g.breaks[b + 1]) ++b;
        lut[2 + i] = (uint8_t)((x >= g.breaks.front() && b < g.count) ? b : g.count);
      }
      // Is the table an affine map followed by a shift?  For every multiplier near 65536 * buckets / span the
      // codes' constraints  lut[c] * 65536 <= c * mul + add < (lut[c] + 1) * 65536  leave an interval for add.
      {
        bool covered = true;   // every code of the domain falls into a bucket
        for (int64_t c = 2; c < entries; ++c) covered = covered && lut[(size_t)c] < g.count;
        const int64_t span = (int64_t)g.breaks.back() - g.breaks.front();
        if (covered && span > 0) {
          const int64_t m0 = (int64_t)std::llround(65536.0 * g.count / (double)span);
          for (int64_t dm = 0; dm <= 256 && !g.arith; ++dm)
            for (int sgn = 0; sgn < (dm ? 2 : 1) && !g.arith; ++sgn) {
              const int64_t mul = m0 + (sgn ? -dm : dm);
              if (mul <= 0) continue;
              int64_t lo = INT64_MIN, hi = INT64_MAX;   // add in [lo, hi]
              for (int64_t c = 2; c < entries; ++c) {
                lo = std::max(lo, (int64_t)lut[(size_t)c] * 65536 - c * mul);
                hi = std::min(hi, ((int64_t)lut[(size_t)c] + 1) * 65536 - 1 - c * mul);
              }
              if (lo > hi) continue;
              const int64_t add = lo + (hi - lo) / 2;
              if (entries * mul + std::llabs(add) >= (int64_t)1 << 31 || 2 * mul + add < 0) continue;
              g.arith = true;
              g.arMul = (int32_t)mul;
              g.arAdd = (int32_t)add;
            }
          // the same search with the two staged special codes among the constraints
          const int64_t oorCode = entries, nanCode = 65535;
          for (int64_t dm = 0; dm <= 256 && !g.clampFit && oorCode < nanCode; ++dm)
            for (int sgn = 0; sgn < (dm ? 2 : 1) && !g.clampFit; ++sgn) {
              const int64_t mul = m0 + (sgn ? -dm : dm);
              if (mul <= 0) continue;
              int64_t lo = INT64_MIN, hi = INT64_MAX;
              for (int64_t c = 2; c <= entries; ++c) {
                const int64_t want = c < entries ? (int64_t)lut[(size_t)c] : (int64_t)g.count;
                lo = std::max(lo, want * 65536 - c * mul);
                hi = std::min(hi, (want + 1) * 65536 - 1 - c * mul);
              }
              lo = std::max(lo, ((int64_t)g.count + 1) * 65536 - nanCode * mul);   // missing input: at least count + 1
              if (lo > hi) continue;
              const int64_t add = lo + (hi - lo) / 2;
              if (nanCode * mul + std::llabs(add) >= (int64_t)1 << 31 || 2 * mul + add < 0) continue;
              g.clampFit = true;
              g.clMul = (int32_t)mul;
              g.clAdd = (int32_t)add;
            }
        }
      }
      auto li = lutOf.emplace(lut, (int32_t)p.lut.size());
      if (li.second) p.lut.insert(p.lut.end(), lut.begin(), lut.end());
      g.lutOffset = li.first->second;
    }
  }
  // features all of whose discrete leaves can bucket arithmetically with clamped special codes
  {
    std::vector<int8_t> all(F, 1), any(F, 0);
    for (const IndexGroup& g : p.groups) {
      any[g.feature] = 1;
      if (!(g.mode == kLut && g.clampFit)) all[g.feature] = 0;
    }
    for (int32_t f = 0; f < F; ++f) p.features[f].clampCodes = any[f] && all[f] && p.features[f].codeSlot >= 0;
  }
  // a feature whose code array is unused (all its groups generic) needs no code slot; harmless to keep
  for (size_t v = 0; v < n; ++v) {
    if (d.group[v] < 0) continue;
    const IndexGroup& g = p.groups[d.group[v]];
    const FeatureMeta& fm = p.features[g.feature];
    const int32_t count = g.count;
    const double neg = logSpace ? -INFINITY : 0.0;
    const double nanv = p.marginal ? (logSpace ? 0.0 : 1.0) : neg;
    auto value = [&](int32_t i) {
      double pr = d.tab[d.tabPtr[v] + i];
      return logSpace ? std::log2(pr) : pr;
    };
    p.tabOffset[v] = (int32_t)(logSpace ? p.tabF32.size() : p.tabF64.size());
    auto push = [&](double val) {
      if (logSpace) p.tabF32.push_back((float)val);
      else p.tabF64.push_back(val);
    };
    if (g.mode == kDirect) {
      push(nanv);
      push(neg);
      int32_t b = 0;
      for (int32_t i = 0; i < fm.domain; ++i) {
        int64_t x = (int64_t)fm.lo + i;
        if (!g.histogram) {
          push(x >= 0 && x < count ? value((int32_t)x) : neg);
        } else {
          while (b < count && x >= g.breaks[b + 1]) ++b;
          push((x >= g.breaks.front() && b < count) ? value(b) : neg);
        }
      }
    } else {
      for (int32_t i = 0; i < count; ++i) push(value(i));
      push(neg);
      push(nanv);
    }
  }

  // ---- statistics -----------------------------------------------------------------------------
  PlanStats& s = p.stats;
  s.modelNodes = (int64_t)m.numNodes();
  s.nodes = (int64_t)n;
  std::vector<int32_t> depth(n, 0);
  for (size_t v = 0; v < n; ++v) {
    int64_t k = d.childPtr[v + 1] - d.childPtr[v];
    for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) depth[v] = std::max(depth[v], depth[d.childIdx[e]] + 1);
    switch (d.kind[v]) {
      case kProduct: s.products++; s.productEdges += k; s.opsFp32 += k - 1; s.opsFp64 += k - 1; break;
      case kSum: s.sums++; s.sumEdges += k; s.opsSfu += k + 1; s.opsFp32 += 4 * k - 1; s.opsFp64 += 2 * k - 1; break;
      case kGaussian: s.gauss++; s.opsFp32 += 3; s.opsFp64 += 1; break;
      case kCategorical: s.cats++; s.opsFp32 += 2; s.opsFp64 += 1; break;
      default: s.hists++; s.opsFp32 += 2; s.opsFp64 += 1; break;
    }
  }
  s.opsFp32 += s.opsSfu;
  s.opsFp64 += 40;
  s.depth = depth[n - 1];
  {
    // reference-style statistics on the two-input form: an operand at position i of k sits
    // ceil(log2 k) levels (at most) below its node in the balanced tree; sum operands one more (the
    // multiplication by the weight)
    s.featureCount = d.numFeatures;
    std::vector<int64_t> level(n, -1);
    level[n - 1] = 0;
    std::vector<double> constants;
    for (size_t v = n; v-- > 0;) {
      if (level[v] < 0) continue;
      const int64_t k = d.childPtr[v + 1] - d.childPtr[v];
      if (k == 0) continue;
      int64_t lg = 0;
      while (((int64_t)1 << lg) < k) ++lg;
      const bool sum = d.kind[v] == kSum;
      if (sum) { s.refAdds += k - 1; s.refMuls += k; } else { s.refMuls += k - 1; }
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
        level[d.childIdx[e]] = std::max(level[d.childIdx[e]], level[v] + lg + (sum ? 1 : 0));
        if (sum) constants.push_back(d.weight[e]);
      }
    }
    std::sort(constants.begin(), constants.end());
    s.refConstants = (int64_t)(std::unique(constants.begin(), constants.end()) - constants.begin());
    std::vector<int64_t> leafLevels;
    for (size_t v = 0; v < n; ++v)
      if (d.childPtr[v + 1] == d.childPtr[v] && level[v] >= 0) leafLevels.push_back(level[v]);
    if (!leafLevels.empty()) {
      std::sort(leafLevels.begin(), leafLevels.end());
      s.minDepth = leafLevels.front();
      s.maxDepth = leafLevels.back();
      double acc = 0.0;
      for (int64_t l : leafLevels) acc += (double)l;
      s.averageDepth = acc / (double)leafLevels.size();
      const size_t h = leafLevels.size() / 2;
      s.medianDepth = leafLevels.size() % 2 ? (double)leafLevels[h] : 0.5 * (double)(leafLevels[h - 1] + leafLevels[h]);
    }
  }
  s.bytesPerSample = (int64_t)m.numFeatures * m.ftype.bytes() + (logSpace ? 4 : 8);

  buildProgram(p, INT32_MAX);
  return p;
}

// Interpreter program with liveness-based value slots.  Slots [0, smemSlots) live in shared memory,
// the rest in a per-CTA scratch area in global memory.  A value whose live range is much longer than
// the shared-memory capacity goes to scratch straight away: it would pin a slot that many short-lived
// values could share.
void buildProgram(Plan& p, int32_t smemSlots) {
  const Dag& d = p.dag;
  const size_t n = d.size();
  const double LOG2E = 1.4426950408889634074;
  p.prog.clear();
  p.progConsts.clear();
  const bool lin = !p.logSpace;
  std::map<uint64_t, int32_t> constIndex;   // equal constants share one table entry
  auto constant = [&](double v) -> int32_t {
    uint64_t bits;
    std::memcpy(&bits, &v, 8);
    auto ins = constIndex.emplace(bits, (int32_t)p.progConsts.size());
    if (ins.second) p.progConsts.push_back(v);
    return ins.first->second;
  };
  std::vector<int64_t> lastUse(n, -1);
  for (size_t v = 0; v < n; ++v)
    for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) lastUse[d.childIdx[e]] = (int64_t)v;
  const bool limited = smemSlots != INT32_MAX;
  const int64_t longRange = limited ? 8ll * smemSlots : INT64_MAX;
  std::vector<int32_t> slot(n, -1), remaining(d.uses);
  std::vector<int32_t> freeSmem, freeGlobal;
  int32_t nSmem = 0, nGlobal = 0;
  for (size_t v = 0; v < n; ++v) {
    int64_t lo = d.childPtr[v], hi = d.childPtr[v + 1];
    // operands are read before the result is written, so a dying operand's slot may be reused
    for (int64_t e = lo; e < hi; ++e) {
      int32_t c = d.childIdx[e];
      if (--remaining[c] == 0) (slot[c] < smemSlots ? freeSmem : freeGlobal).push_back(slot[c]);
    }
    int32_t dst = -1;
    const bool preferGlobal = limited && lastUse[v] - (int64_t)v > longRange;
    if (!preferGlobal) {
      if (!freeSmem.empty()) { dst = freeSmem.back(); freeSmem.pop_back(); }
      else if (nSmem < smemSlots) dst = nSmem++;
    }
    if (dst < 0) {
      if (!freeGlobal.empty()) { dst = freeGlobal.back(); freeGlobal.pop_back(); }
      else dst = smemSlots + nGlobal++;
    }
    slot[v] = dst;
    switch (d.kind[v]) {
      case kGaussian: {
        double sd = d.stddev[v];
        p.prog.push_back(OP_GAUSS);
        p.prog.push_back(dst);
        p.prog.push_back(p.features[d.feature[v]].valueSlot);
        if (lin) {
          const double var = sd * sd;
          p.prog.push_back(constant(d.mean[v]));
          p.prog.push_back(constant(-1.0 / (2.0 * var)));
          p.prog.push_back(constant(1.0 / std::sqrt(2.0 * M_PI * var)));
          break;
        }
        p.prog.push_back((int32_t)f32bits((float)d.mean[v]));
        p.prog.push_back((int32_t)f32bits((float)(-(1.0 / (2.0 * sd * sd)) * LOG2E)));
        p.prog.push_back((int32_t)f32bits((float)((-std::log(sd) - 0.5 * std::log(2 * M_PI)) * LOG2E)));
        break;
      }
      case kCategorical:
      case kHistogram: {
        const IndexGroup& g = p.groups[d.group[v]];
        if (g.mode == kGeneric) {
          p.prog.push_back(OP_HISTG);
          p.prog.push_back(dst);
          p.prog.push_back(p.features[g.feature].valueSlot);
          p.prog.push_back(g.brkOffset);
          p.prog.push_back(g.count);
          p.prog.push_back(p.tabOffset[v]);
        } else {
          p.prog.push_back(OP_TABLE);
          p.prog.push_back(dst);
          p.prog.push_back(p.features[g.feature].codeSlot);
          p.prog.push_back(g.lutOffset);
          p.prog.push_back(p.tabOffset[v]);
        }
        break;
      }
      case kProduct:
        p.prog.push_back(OP_PROD);
        p.prog.push_back(dst);
        p.prog.push_back((int32_t)(hi - lo));
        for (int64_t e = lo; e < hi; ++e) p.prog.push_back(slot[d.childIdx[e]]);
        break;
      default:
        p.prog.push_back(OP_SUM);
        p.prog.push_back(dst);
        p.prog.push_back((int32_t)(hi - lo));
        for (int64_t e = lo; e < hi; ++e) {
          p.prog.push_back(slot[d.childIdx[e]]);
          p.prog.push_back(lin ? constant(d.weight[e]) : (int32_t)f32bits((float)std::log2(d.weight[e])));
        }
        break;
    }
    }
  p.prog.push_back(OP_END);
  p.prog.push_back(slot[n - 1]);
  if (!limited) p.numSlots = nSmem;
  p.numSmemSlots = nSmem;
  p.numSpillSlots = nGlobal;
}

}  // namespace spnb
