#include "emit.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <sstream>

namespace spnb {

namespace {

std::string lit32(float f) {
  if (std::isinf(f)) return f < 0 ? "NEG_INF" : "POS_INF";
  char buf[64];
  std::snprintf(buf, sizeof buf, "%af", (double)f);
  return buf;
}
std::string lit64(double f) {
  if (std::isinf(f)) return f < 0 ? "(-POS_INF)" : "POS_INF";
  char buf[64];
  std::snprintf(buf, sizeof buf, "%a", f);
  return buf;
}

const char* inputCType(const FeatureType& t) {
  if (t.kind == InKind::Float) return t.bits == 32 ? "float" : "double";
  bool u = t.kind == InKind::UInt;
  switch (t.bits) {
    case 8: return u ? "unsigned char" : "signed char";
    case 16: return u ? "unsigned short" : "short";
    case 32: return u ? "unsigned int" : "int";
    default: return u ? "unsigned long long" : "long long";
  }
}

// balanced binary combination of terms: ((a op b) op (c op d)) for instruction-level parallelism
std::string balanced(const std::vector<std::string>& t, size_t lo, size_t hi, const std::function<std::string(const std::string&, const std::string&)>& comb) {
  if (hi - lo == 1) return t[lo];
  size_t mid = lo + (hi - lo + 1) / 2;
  return comb(balanced(t, lo, mid, comb), balanced(t, mid, hi, comb));
}

// maximum of the terms as a tree of three-input max instructions (sm_100 has max.f32 d, a, b, c)
std::string max3Tree(const std::vector<std::string>& t, size_t lo, size_t hi) {
  size_t k = hi - lo;
  if (k == 1) return t[lo];
  if (k == 2) return "fmaxf(" + t[lo] + ", " + t[lo + 1] + ")";
  if (k == 3) return "max3(" + t[lo] + ", " + t[lo + 1] + ", " + t[lo + 2] + ")";
  size_t a = lo + (k + 2) / 3, b = a + (k - (k + 2) / 3 + 1) / 2;
  return "max3(" + max3Tree(t, lo, a) + ", " + max3Tree(t, a, b) + ", " + max3Tree(t, b, hi) + ")";
}

}  // namespace

// Bytes of the code -> bucket byte tables the generated kernel reads: none if every table-driven group's
// buckets are computed arithmetically.
static size_t lutBytesNeeded(const Plan& p, const EmitOptions& opt, bool clamp) {
  for (const IndexGroup& g : p.groups)
    if (g.mode == kLut && !(g.arith && opt.bucketArith) && !(clamp && p.features[g.feature].clampCodes)) return p.lut.size();
  return 0;
}

std::string emitCuda(const Plan& p, const EmitOptions& opt, EmitInfo* info) {
  const Dag& d = p.dag;
  const size_t n = d.size();
  const bool lg = p.logSpace;
  const char* real = lg ? "float" : "double";
  const int F = d.numFeatures;
  size_t tabEntries = lg ? p.tabF32.size() : p.tabF64.size();
  const size_t realBytes = lg ? 4 : 8;
  // ---- fused leaf tables ---------------------------------------------------------------------------------
  // A product's discrete leaf children over distinct features, each read through a (domain + 2)-entry table,
  // are looked up together: one table over the combined code  c1 + S1 * (c2 + S2 * c3)  holds the product of
  // the leaves' values (the sum of their logarithms), so k leaves cost one table read and k - 1 integer
  // multiply-adds instead of k reads and k - 1 floating-point operations.  Small discrete models are bound by
  // the shared-memory pipe (two wavefronts per 64-bit table read), not by arithmetic.  Only for kernels of one
  // function whose tables, the fused ones included, stay resident in shared memory; a leaf with another
  // consumer keeps its own read.  The fused tables follow the plan's tables in the table image.
  struct FusedGroup { std::vector<int32_t> leaves; long long offset = 0; };
  std::vector<FusedGroup> fused;
  std::vector<int32_t> fusedHead(n, -1);     // leaf -> its group, for the group's first leaf in evaluation order
  std::vector<uint8_t> fusedAway(n, 0);      // leaf evaluated by its group's first leaf
  std::vector<double> fusedTable;
  {
    const size_t cn = opt.chunkNodes > 0 ? (size_t)opt.chunkNodes : n;
    const bool oneFunction = opt.chunkExact ? n <= cn : n <= cn + cn / 2;
    const size_t cap = (size_t)opt.smemTableLimit / realBytes;
    if (opt.fuseLeaves != 0 && oneFunction && opt.scoped != 1 && !opt.bucketClamp && tabEntries > 0 && tabEntries < cap) {
      std::vector<int32_t> uses(n, 0);
      for (size_t v = 0; v < n; ++v)
        for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) ++uses[d.childIdx[e]];
      auto entriesOf = [&](int32_t c) -> long long {
        if (d.kind[c] != kCategorical && d.kind[c] != kHistogram) return 0;
        const IndexGroup& G = p.groups[d.group[c]];
        if (G.mode != kDirect || uses[c] != 1 || p.tabOffset[c] < 0) return 0;
        return (long long)p.features[G.feature].domain + 2;
      };
      const long long maxEntries = std::max(opt.fuseEntries, 4);
      for (size_t v = 0; v < n; ++v) {
        if (d.kind[v] != kProduct) continue;
        FusedGroup g;
        long long size = 1;
        auto close = [&]() {
          if (g.leaves.size() >= 2 && tabEntries + fusedTable.size() + (size_t)size <= cap) {
            g.offset = (long long)(tabEntries + fusedTable.size());
            // entry of the combined code: leaf 0's code runs fastest
            for (long long idx = 0; idx < size; ++idx) {
              long long rest = idx;
              double acc = lg ? 0.0 : 1.0;
              for (int32_t c : g.leaves) {
                const long long sz = entriesOf(c), code = rest % sz;
                rest /= sz;
                const double t = lg ? (double)p.tabF32[(size_t)p.tabOffset[c] + (size_t)code] : p.tabF64[(size_t)p.tabOffset[c] + (size_t)code];
                acc = lg ? acc + t : acc * t;
              }
              fusedTable.push_back(acc);
            }
            int32_t head = *std::min_element(g.leaves.begin(), g.leaves.end());
            fusedHead[head] = (int32_t)fused.size();
            for (int32_t c : g.leaves) if (c != head) fusedAway[c] = 1;
            fused.push_back(g);
          }
          g.leaves.clear();
          size = 1;
        };
        for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
          const int32_t c = d.childIdx[e];
          const long long sz = entriesOf(c);
          if (sz == 0) continue;
          if (size * sz > maxEntries) close();
          g.leaves.push_back(c);
          size *= sz;
        }
        close();
      }
      tabEntries += fusedTable.size();
    }
  }
  // Launch shape.  The body is far larger than the instruction caches, so the warps of an SM should
  // walk it together: few, large CTAs (their warps leave the staging barrier at the same time), and
  // 1024 resident threads per SM at <= 64 registers when the staged inputs of that many samples fit
  // into shared memory; otherwise the largest CTA of the candidate list below that fits, alone on its SM.
  int TILE = opt.tile, minBlocks = opt.minBlocksPerSM;
  // staged codes are bytes when every discrete feature's domain (+ the two special codes) fits
  int maxDomain = 0;
  for (const FeatureMeta& fm : p.features)
    if (fm.codeSlot >= 0) maxDomain = std::max(maxDomain, fm.domain);
  // arithmetic buckets with clamped special codes: the missing-input code 65535 needs 16-bit codes
  const bool clampAllowed = opt.bucketClamp;
  bool anyClamp = false;
  for (const FeatureMeta& fm : p.features) anyClamp = anyClamp || (clampAllowed && fm.clampCodes);
  const int cb = (maxDomain + 2 <= 255 && !anyClamp) ? 1 : 2;
  const size_t tabBytes = tabEntries * realBytes;
  size_t tableLimit = (size_t)opt.smemTableLimit;
  if (TILE <= 0) {
    const bool nanFlags = p.marginal && p.ftype.isFloat() && p.numValueSlots > 0 && p.stats.gauss > 0;
    const size_t perThread = (size_t)p.numValueSlots * realBytes + (size_t)p.numCodeSlots * cb + (nanFlags ? 4 : 0);
    size_t fixed = (size_t)d.numFeatures * 16 + 64;
    if (lutBytesNeeded(p, opt, clampAllowed) <= (size_t)opt.smemTableLimit) fixed += lutBytesNeeded(p, opt, clampAllowed);
    const size_t budget = 226 * 1024;  // one CTA may use up to 227 KB
    bool found = false;
    // candidates in steps of a warp below 512 threads: with 1 KB of staged inputs per sample the difference
    // between 256 and 320 samples per CTA is a tenth of the run time (all warps of a CTA share every fetched
    // instruction)
    static const int kTiles[] = {1024, 768, 512, 448, 384, 352, 320, 288, 256, 224, 192, 160, 128, 96, 64};
    for (int cand : kTiles) {
      for (size_t w = (size_t)opt.smemTableLimit; w >= std::min<size_t>(8192, (size_t)opt.smemTableLimit) && !found; w /= 2) {
        // a larger CTA with a smaller table window beats a smaller CTA
        if (fixed + std::min(tabBytes, w) + 16 + (size_t)(cand + 1) * perThread <= budget) {
          tableLimit = w;
          TILE = cand;
          found = true;
        }
      }
      if (found) break;
    }
    if (!found) TILE = 64;
    if (minBlocks <= 0) {
      minBlocks = 1;
      // A small model's code stays in the instruction cache, so nothing is gained by 32 warps walking it together;
      // two CTAs of 512 threads per SM then do better than one of 1024: one stages or waits at a barrier while the
      // other evaluates, and a batch's last round of tiles is half as coarse (352-node model, 1 M samples: 59.0 µs
      // with one CTA of 1024 threads per SM, 55.2 with two of 512; a 2 000-node model loses 2 % that way).  Taken
      // when both CTAs fit with either staging scheme (two buffers of raw rows, or staged slots plus tables).
      const size_t half = (233472 / 2 - 1024);
      const size_t rowsAsync = 2 * (((size_t)512 * (size_t)(d.numFeatures | 1) * 4 + 15) & ~size_t(15)) + 64;
      const size_t rowsSync = fixed + 16 + (size_t)513 * perThread;
      if (TILE == 1024 && n <= 1000 && opt.scoped != 1 && tabBytes <= (size_t)opt.smemTableLimit &&
          std::max(rowsAsync, rowsSync) + tabBytes + 64 <= half) {
        TILE = 512;
        minBlocks = 2;
      }
    }
  } else if (minBlocks <= 0) {
    minBlocks = std::max(1, 1024 / TILE);
  }
  // ---- scope-local staging (see EmitOptions::scoped) ---------------------------------------------------
  // DAGs up to one and a half chunk sizes stay in one function; larger ones are cut into equal stretches
  size_t chunkNodes = opt.chunkNodes > 0 ? (size_t)opt.chunkNodes : n;
  if (!opt.chunkExact) {
    if (n <= chunkNodes + chunkNodes / 2) chunkNodes = n;
    else chunkNodes = (n + (n + chunkNodes - 1) / chunkNodes - 1) / ((n + chunkNodes - 1) / chunkNodes);
  }
  const bool scopedPossible = lg && p.ftype.isFloat() && p.ftype.bits == 32;
  const bool scoped = scopedPossible &&
                      (opt.scoped == 1 || (opt.scoped < 0 && opt.tile <= 0 && TILE < 1024 && n > chunkNodes));
  if (scoped) {
    TILE = opt.tile > 0 ? opt.tile : 1024;
    minBlocks = 1;
    tableLimit = std::min<size_t>((size_t)opt.smemTableLimit, 32 * 1024);
  }
  const int SX = scoped ? TILE : TILE + 1;   // the transposing store of the row-major path needs the padding
  // scope-local staging: the discrete features' codes come ready-made from a plane behind the feature-major copy
  const bool codePlane = scoped && opt.codePlane != 0 && p.numCodeSlots > 0;
  // Leaf tables are always read from shared memory.  Tables larger than the window are streamed
  // through it: leaves appear in the body in table order, so at the points where the next leaf's
  // table lies beyond the window the CTA reloads the window from global memory between two barriers.
  const bool tabSmem = tabEntries > 0;
  const bool streamed = tabBytes > tableLimit;
  if (streamed && !fused.empty()) {
    // the fused tables do not follow the leaves' order, which a streamed window relies on: emit without them
    EmitOptions plain = opt;
    plain.fuseLeaves = 0;
    return emitCuda(p, plain, info);
  }
  const size_t winBytes = streamed ? (tableLimit & ~size_t(15)) : ((tabBytes + 15) & ~size_t(15));
  const bool floatIn = p.ftype.isFloat();
  const double LOG2E = 1.4426950408889634074;
  const int NV = p.numValueSlots, NC = p.numCodeSlots;
  bool identity = (NC == 0 && NV == F) && !scoped;
  for (int f = 0; identity && f < F; ++f) identity = p.features[f].valueSlot == f;
  const size_t lutBytes = lutBytesNeeded(p, opt, clampAllowed);
  const bool lutSmem = lutBytes > 0 && lutBytes <= (size_t)opt.smemTableLimit;
  // ---- asynchronous double-buffered staging (see EmitOptions::asyncStage) -----------------------------------
  const int RS = F | 1;                                      // row stride in words: odd, conflict-free
  const size_t asyncBuf = ((size_t)TILE * RS * 4 + 15) & ~size_t(15);
  // every input is read as a value by Gaussian leaves (no staged codes, no leaf tables): the body indexes a
  // staged row by the feature itself
  // ... or the model has discrete leaves whose tables stay resident in shared memory: the rows are staged raw
  // (32-bit inputs), every body function digests the discrete features it reads into codes once, in registers
  // (at most 27 features fit two buffers of 1024 rows), and the tables sit behind the two buffers
  bool asyncDiscrete = NC > 0 && !anyClamp && !streamed && (lutBytes == 0 || lutSmem) && (lg ? floatIn || NV == 0 : NV == 0);
  for (const IndexGroup& g : p.groups) asyncDiscrete = asyncDiscrete && g.mode != kGeneric;
  const size_t asyncTables = (tabSmem ? winBytes : 0) + (lutSmem ? p.lut.size() + 4 : 0) + 32;
  const bool asyncStage = opt.asyncStage != 0 && !scoped && p.ftype.bits == 32 && opt.groupTiles <= 1 &&
                          ((NC == 0 && NV > 0 && tabEntries == 0 && lg && floatIn) || asyncDiscrete) &&
                          2 * asyncBuf + 64 + asyncTables <= 226 * 1024;
  const bool nanFlagsWanted = p.marginal && floatIn && NV > 0 && p.stats.gauss > 0;

  // ---- chunks: consecutive stretches of the evaluation order, one generated function each -----------------
  // Row-major path: equal stretches of chunkNodes nodes, every chunk reads the tile's inputs staged once.
  // Scoped path: a stretch also ends where its leaves would need more staged bytes per sample than fit.
  std::vector<size_t> chunkStart{0};
  std::vector<int32_t> chunkOf(n, 0);
  // per chunk: staged features (values, then codes) and, per node, the slot its leaf reads
  std::vector<std::vector<int32_t>> chunkValueFeat, chunkCodeFeat;
  std::vector<int32_t> leafSlot(n, -1);
  size_t scopeBudget = 0, maxStageBytes = 0, maxValueFeat = 0, maxCodeFeat = 0;
  bool fixedCodeBase = false;
  if (!scoped) {
    for (size_t v = chunkNodes; v < n; v += chunkNodes) chunkStart.push_back(v);
    for (size_t v = 0; v < n; ++v) chunkOf[v] = (int32_t)(v / chunkNodes);
  } else {
    const size_t fixed = 64 + std::min(tabBytes, tableLimit) + 16 + (lutSmem ? p.lut.size() + 4 : 0);
    scopeBudget = (226 * 1024 - fixed) / (size_t)TILE - (nanFlagsWanted ? 4 : 0) - (size_t)std::max(opt.prefetchSlots, 0) * 4;
    if (opt.scopeBytes > 0) scopeBudget = std::min<size_t>(scopeBudget, (size_t)opt.scopeBytes);
    // Values alive across position q (defined before q, used at or after q): what a cut at q sends through
    // the scratch area.  A chunk is grown until its leaves would need more staged bytes than fit (or it has
    // chunkNodes nodes); with scopeCut = 1 the cut is then moved back to the position of its second half where
    // the fewest values cross, which is where one sub-DAG ends and the next begins in the depth-first order.
    std::vector<int32_t> crossing(n + 1, 0);
    {
      std::vector<int64_t> last(n, -1);
      for (size_t v = 0; v < n; ++v)
        for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) last[d.childIdx[e]] = (int64_t)v;
      std::vector<int32_t> diff(n + 2, 0);
      for (size_t u = 0; u < n; ++u)
        if (last[u] > (int64_t)u) { diff[u + 1]++; diff[(size_t)last[u] + 1]--; }   // alive at positions u+1 .. last[u]
      int32_t run = 0;
      for (size_t q = 0; q <= n; ++q) { run += diff[q]; crossing[q] = run; }
    }
    auto needOf = [&](size_t v, int32_t& needValue, int32_t& needCode) {
      needValue = needCode = -1;
      if (d.kind[v] == kGaussian) needValue = d.feature[v];
      else if (d.kind[v] == kCategorical || d.kind[v] == kHistogram) {
        const IndexGroup& G = p.groups[d.group[v]];
        if (G.mode == kGeneric) needValue = G.feature; else needCode = G.feature;
      }
    };
    // Without CTA-wide barriers between the chunks (chunkBarrier = 0) a warp may stage its next chunk while
    // another still evaluates the current one.  A thread's staged words and bytes must then never share an address
    // with another thread's, whatever the two chunks stage: values (words) and codes (bytes / half-words) get
    // separate areas with one boundary for all chunks, and separate budgets in proportion to the model's features.
    size_t valueBudget = scopeBudget, codeBudget = scopeBudget;
    const bool splitAreas = opt.chunkBarrier == 0;
    if (splitAreas) {
      size_t fv = 0, fc = 0;
      for (int f = 0; f < F; ++f) { fv += p.features[f].valueSlot >= 0; fc += p.features[f].codeSlot >= 0; }
      if (fv && fc) {
        valueBudget = std::max<size_t>(4, scopeBudget * (4 * fv) / (4 * fv + (size_t)cb * fc) / 4 * 4);
        codeBudget = std::max<size_t>((size_t)cb, scopeBudget - valueBudget);
      }
    }
    std::vector<int32_t> vstamp(F, -1), cstamp(F, -1), vslotOf(F, -1), cslotOf(F, -1);
    chunkStart.clear();
    int32_t cur = 0, stamp = 0;
    size_t begin = 0;
    while (begin < n) {
      // how far the budget reaches
      ++stamp;
      size_t bytes = 0, vbytes = 0, cbytes = 0, reach = begin;
      for (; reach < n && reach - begin < chunkNodes; ++reach) {
        int32_t nv, nc;
        needOf(reach, nv, nc);
        size_t addV = 0, addC = 0;
        if (nv >= 0 && vstamp[nv] != stamp) addV = 4;
        if (nc >= 0 && cstamp[nc] != stamp) addC = (size_t)cb;
        if (reach > begin && (bytes + addV + addC > scopeBudget ||
                              (splitAreas && (vbytes + addV > valueBudget || cbytes + addC > codeBudget)))) break;
        if (nv >= 0) vstamp[nv] = stamp;
        if (nc >= 0) cstamp[nc] = stamp;
        bytes += addV + addC;
        vbytes += addV;
        cbytes += addC;
      }
      size_t cut = reach;
      if (reach < n && opt.scopeCut == 1) {
        const size_t lo = begin + std::max<size_t>(1, (reach - begin) / 2);
        for (size_t q = lo; q <= reach; ++q)
          if (crossing[q] <= crossing[cut]) cut = q;
      }
      // the chunk [begin, cut): its staged features and the slot every leaf reads
      chunkStart.push_back(begin);
      chunkValueFeat.emplace_back();
      chunkCodeFeat.emplace_back();
      ++stamp;
      for (size_t v = begin; v < cut; ++v) {
        chunkOf[v] = cur;
        int32_t nv, nc;
        needOf(v, nv, nc);
        if (nv >= 0) {
          if (vstamp[nv] != stamp) {
            vstamp[nv] = stamp;
            vslotOf[nv] = (int32_t)chunkValueFeat.back().size();
            chunkValueFeat.back().push_back(nv);
          }
          leafSlot[v] = vslotOf[nv];
        }
        if (nc >= 0) {
          if (cstamp[nc] != stamp) {
            cstamp[nc] = stamp;
            cslotOf[nc] = (int32_t)chunkCodeFeat.back().size();
            chunkCodeFeat.back().push_back(nc);
          }
          leafSlot[v] = cslotOf[nc];
        }
      }
      ++cur;
      begin = cut;
    }
    for (size_t c = 0; c < chunkValueFeat.size(); ++c) {
      maxStageBytes = std::max(maxStageBytes, chunkValueFeat[c].size() * 4 + chunkCodeFeat[c].size() * (size_t)cb);
      maxValueFeat = std::max(maxValueFeat, chunkValueFeat[c].size());
      maxCodeFeat = std::max(maxCodeFeat, chunkCodeFeat[c].size());
    }
    if (splitAreas) { fixedCodeBase = true; maxStageBytes = maxValueFeat * 4 + maxCodeFeat * (size_t)cb; }
  }
  chunkStart.push_back(n);
  const size_t nChunks = chunkStart.size() - 1;
  // byte offset of a chunk's staged codes behind its staged values (scoped path)
  auto codeBase = [&](size_t c) { return (fixedCodeBase ? maxValueFeat : chunkValueFeat[c].size()) * (size_t)4 * SX; };
  // Gaussian leaves of a query with marginal support must turn a NaN input into log 1 = 0: a compare
  // and a select per leaf.  NaNs are rare in practice, so the body is emitted twice: a plain version
  // and a NaN-aware one; a CTA takes the second only if one of its samples has a NaN among the staged
  // values (flagged per row while the tile is staged).
  const bool twoBodies = p.marginal && floatIn && NV > 0 && p.stats.gauss > 0;

  // shared memory layout (bytes): [fm int4 x NF] [xs real x NV*SX] [cs u8|u16 x NC*SX] [tab] [lut] [nan flags int x TILE]
  const size_t offFm = 0;
  const size_t offXs = (identity || scoped) ? 0 : (size_t)F * 16;
  const size_t offCs = offXs + (size_t)NV * SX * realBytes;
  const size_t offTab = asyncStage ? 2 * asyncBuf
                        : scoped ? ((maxStageBytes * SX + 15) & ~size_t(15)) : ((offCs + (size_t)NC * SX * cb + 15) & ~size_t(15));
  const size_t offLut = offTab + (tabSmem ? winBytes : 0);
  const size_t offNan = (offLut + (lutSmem ? p.lut.size() : 0) + 3) & ~size_t(3);
  // scope-local staging with an operand ring: [slot][TILE] floats behind everything else
  const int pfSlots = scoped && lg ? std::max(opt.prefetchSlots, 0) : 0;
  const size_t offPf = (offNan + 15) & ~size_t(15);
  const size_t smemTotal = pfSlots > 0 ? offPf + (size_t)pfSlots * TILE * 4
                                       : offNan + ((twoBodies && !scoped && !asyncStage) ? (size_t)TILE * 4 : 0);

  std::ostringstream o;
  o << "// generated by spnb: straight-line joint log-likelihood kernel, one thread per sample\n";
  o << "typedef " << inputCType(p.ftype) << " in_t;\n";
  o << "typedef " << real << " real_t;\n";
  o << "typedef " << real << " out_t;\n";
  o << "#define NEG_INF __int_as_float(0xff800000)\n#define POS_INF __int_as_float(0x7f800000)\n";
  o << "#define NF " << F << "\n#define TILE " << TILE << "\n#define SX " << SX << "\n";
  o << "#define NTAB " << tabEntries << "\n#define NLUT " << p.lut.size() << "\n";
  o << "static __device__ __forceinline__ float ex2(float x){float y;asm(\"ex2.approx.ftz.f32 %0, %1;\":\"=f\"(y):\"f\"(x));return y;}\n";
  o << "static __device__ __forceinline__ float max3(float a, float b, float c){float y;asm(\"max.ftz.f32 %0, %1, %2, %3;\":\"=f\"(y):\"f\"(a),\"f\"(b),\"f\"(c));return y;}\n";
  o << "static __device__ __forceinline__ float lg2(float x){float y;asm(\"lg2.approx.ftz.f32 %0, %1;\":\"=f\"(y):\"f\"(x));return y;}\n";
  if (!identity) {
    o << "// per feature: lo, domain, code slot, value slot\n__device__ const int FM[NF * 4] = {";
    for (int f = 0; f < F; ++f) {
      const FeatureMeta& fm = p.features[f];
      // (code slot + 65536: the feature's special codes are the clamped ones, see FeatureMeta::clampCodes)
      o << (f ? "," : "") << fm.lo << "," << fm.domain << ","
        << (fm.codeSlot >= 0 && clampAllowed && fm.clampCodes ? fm.codeSlot + 65536 : fm.codeSlot) << "," << fm.valueSlot;
    }
    o << "};\n";
  }
  // saturating conversion of one raw input to int (truncation toward zero for floating inputs)
  if (floatIn) o << "#define TOINT(v) " << (p.ftype.bits == 32 ? "__float2int_rz(v)" : "__double2int_rz(v)") << "\n";
  else if (p.ftype.bits == 64 && p.ftype.kind == InKind::Int) o << "#define TOINT(v) ((v) > 2147483647ll ? 2147483647 : ((v) < -2147483648ll ? (-2147483647 - 1) : (int)(v)))\n";
  else if (p.ftype.bits == 64) o << "#define TOINT(v) ((v) > 2147483647ull ? 2147483647 : (int)(v))\n";
  else if (p.ftype.bits == 32 && p.ftype.kind == InKind::UInt) o << "#define TOINT(v) ((v) > 2147483647u ? 2147483647 : (int)(v))\n";
  else o << "#define TOINT(v) ((int)(v))\n";
  // Shared-memory reads are emitted as asm statements on 32-bit shared addresses with the constant
  // part of the address written into the instruction text.  To the optimiser they are pure
  // functions of their operands (thousands of ordinary loads through one pointer make its
  // memory-dependence analysis quadratic), and because the text differs per use, two reads of one
  // staged input stay separate instead of pinning a register across the whole body.
  const int rb = (int)realBytes;
  const char* ldReal = lg ? "ld.shared.f32" : "ld.shared.f64";
  const char* cReal = lg ? "f" : "d";
  size_t maxChunkValues = 0;
  for (auto& cv : chunkValueFeat) maxChunkValues = std::max(maxChunkValues, cv.size());
  const bool mergeX = scoped ? maxChunkValues <= 32 : NV <= 32;  // few staged values (Gaussian inputs): identical reads may merge
  auto ldsStmt = [&](const std::string& type, const char* inst, const char* constraint, const std::string& dst,
                     const std::string& base, long long imm, long long uniq) {
    std::ostringstream e;
    e << "  " << type << " " << dst << "; asm(\"" << inst << " %0, [%1+" << imm << "];";
    if (uniq >= 0) e << " // " << uniq;
    e << "\" : \"=" << constraint << "\"(" << dst << ") : \"r\"(" << base << "));\n";
    return e.str();
  };
  auto readX = [&](const std::string& dst, int slot, long long node) {
    return ldsStmt("real_t", ldReal, cReal, dst, "xs_t", asyncStage ? (long long)rb * slot : (long long)rb * slot * SX, mergeX ? -1 : node);
  };
  std::vector<int> featureOfCodeSlot(NC > 0 ? NC : 0, -1);
  for (int f = 0; f < F; ++f)
    if (p.features[f].codeSlot >= 0 && p.features[f].codeSlot < NC) featureOfCodeSlot[p.features[f].codeSlot] = f;
  auto readCode = [&](const std::string& dst, int slot, long long node) {
    // asynchronous staging: the code was digested from the raw row at the top of the function
    if (asyncStage) return "  const int " + dst + " = cf" + std::to_string(featureOfCodeSlot[slot]) + ";\n";
    return ldsStmt("int", cb == 1 ? "ld.shared.u8" : "ld.shared.u16", "r", dst, "cs_t", (long long)cb * slot * SX, node);
  };
  long long winBase = 0;  // first table entry held by the window at the current point of the body
  auto readTab = [&](const std::string& dst, long long off, const std::string& idx, long long node) {
    std::string st = ldsStmt("real_t", ldReal, cReal, dst, "(tab_s + " + std::to_string(rb) + "u * (unsigned)" + idx + ")",
                             (long long)rb * (off - winBase), node);
    // a streamed window changes under the body: its reads must stay between the surrounding barriers
    if (streamed) st.replace(st.find("asm("), 4, "asm volatile(");
    return st;
  };
  auto tableEntriesOf = [&](size_t v) -> long long {
    const IndexGroup& G = p.groups[d.group[v]];
    return G.mode == kDirect ? (long long)p.features[G.feature].domain + 2 : (long long)G.count + 2;
  };
  auto swapWindow = [&](std::ostringstream& out, long long firstEntry) {
    const long long align = 16 / rb;
    winBase = firstEntry / align * align;
    out << "  __syncthreads();\n";
    out << "  { const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(tab_g) + " << winBase * rb << "ll);\n";
    out << "    for (unsigned i = tid; i < " << winBytes / 16 << "u; i += TILE) win[i] = __ldg(src + i); }\n";
    out << "  __syncthreads();\n";
  };
  auto readLut = [&](const std::string& dst, long long off, const std::string& idx, long long node) {
    if (lutSmem) return ldsStmt("int", "ld.shared.u8", "r", dst, "(lut_s + (unsigned)" + idx + ")", off, node);
    std::ostringstream e;
    e << "  int " << dst << "; asm(\"ld.global.nc.u8 %0, [%1+" << off << "]; // " << node << "\" : \"=r\"(" << dst
      << ") : \"l\"(lut_g + " << idx << "));\n";
    return e.str();
  };

  auto emitLeafLookup = [&](std::ostringstream& out, size_t v, const std::string& name) {
    const IndexGroup& G = p.groups[d.group[v]];
    const FeatureMeta& fm = p.features[G.feature];
    const std::string c = "c" + std::to_string(v);
    const int codeSlot = scoped ? leafSlot[v] : fm.codeSlot;
    const int valueSlot = scoped ? leafSlot[v] : (asyncStage ? G.feature : fm.valueSlot);
    if (G.mode == kDirect) {
      out << readCode(c, codeSlot, (long long)v) << readTab(name, p.tabOffset[v], c, (long long)v);
    } else if (G.mode == kLut && clampAllowed && fm.clampCodes) {
      // bucket = min((code * mul + add) >> 16, count + 1): the staged special codes land on the two entries
      // behind the buckets by themselves
      const std::string b = "b" + std::to_string(v);
      out << readCode(c, codeSlot, (long long)v);
      out << "  const int " << b << " = min((" << c << " * " << G.clMul << " + " << G.clAdd << ") >> 16, " << (G.count + 1) << ");\n";
      out << readTab(name, p.tabOffset[v], b, (long long)v);
    } else if (G.mode == kLut && G.arith && opt.bucketArith) {
      // bucket computed from the code; codes 0 (missing input) and 1 (outside the domain) select the two
      // entries behind the buckets
      const std::string b = "b" + std::to_string(v);
      out << readCode(c, codeSlot, (long long)v);
      out << "  const int " << b << " = " << c << " < 2 ? " << (G.count + 1) << " - " << c << " : (" << c << " * " << G.arMul
          << " + " << G.arAdd << ") >> 16;\n";
      out << readTab(name, p.tabOffset[v], b, (long long)v);
    } else if (G.mode == kLut) {
      const std::string b = "b" + std::to_string(v);
      out << readCode(c, codeSlot, (long long)v) << readLut(b, G.lutOffset, c, (long long)v)
          << readTab(name, p.tabOffset[v], b, (long long)v);
    } else {
      std::string xr = "xr" + std::to_string(v), xi = "xi" + std::to_string(v);
      out << readX(xr, valueSlot, (long long)v);
      out << "  const int " << xi << " = " << (lg ? "__float2int_rz" : "__double2int_rz") << "(" << xr << ");\n";
      std::string cnt;
      for (int32_t i = 1; i < G.count; ++i) cnt += (i > 1 ? " + " : "") + std::string("(") + xi + " >= " + std::to_string(G.breaks[i]) + ")";
      if (cnt.empty()) cnt = "0";
      std::string inr = "((" + xi + " >= " + std::to_string(G.breaks.front()) + " && " + xi + " < " + std::to_string(G.breaks.back()) + ") ? (" + cnt + ") : " + std::to_string(G.count) + ")";
      out << "  const int ig" << v << " = ";
      if (floatIn) out << "(" << xr << " != " << xr << ") ? " << (G.count + 1) << " : ";
      out << inr << ";\n";
      out << readTab(name, p.tabOffset[v], "ig" + std::to_string(v), (long long)v);
    }
  };

  // may a node evaluate to -inf (log space)?  decides where the all-(-inf) guard of a sum is needed
  std::vector<uint8_t> mayNeg(n, 0);
  for (size_t v = 0; v < n; ++v) {
    switch (d.kind[v]) {
      case kGaussian: mayNeg[v] = 0; break;
      case kCategorical:
      case kHistogram: mayNeg[v] = 1; break;
      case kProduct:
        for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) mayNeg[v] |= mayNeg[d.childIdx[e]];
        break;
      default: {
        uint8_t all = 1;
        for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) all &= (uint8_t)(mayNeg[d.childIdx[e]] || d.weight[e] == 0.0);
        mayNeg[v] = all;
      }
    }
  }

  auto V = [](int32_t i) { return "v" + std::to_string(i); };
  // ---- chunking.  A DAG with more than chunkNodes nodes is emitted as a sequence of functions over
  // consecutive stretches of the evaluation order (the JIT's time grows much faster than linearly with
  // the size of one function).  A value defined in one chunk and used in a later one travels through a
  // per-CTA scratch area in global memory, [slot][TILE] so that a warp's access is one 128-byte line;
  // slots are reused once their last consumer has run.
  std::vector<int32_t> crossSlot(n, -1);
  int32_t nCross = 0;
  if (nChunks > 1) {
    std::vector<int64_t> lastUse(n, -1);
    std::vector<uint8_t> isCross(n, 0);
    for (size_t v = 0; v < n; ++v)
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
        int32_t c = d.childIdx[e];
        lastUse[c] = std::max<int64_t>(lastUse[c], (int64_t)v);
        if (chunkOf[c] != chunkOf[v]) isCross[c] = 1;
      }
    std::vector<std::vector<int32_t>> dying(n);
    for (size_t v = 0; v < n; ++v)
      if (isCross[v]) dying[(size_t)lastUse[v]].push_back((int32_t)v);
    std::vector<int32_t> freeSlots;
    for (size_t v = 0; v < n; ++v) {
      if (isCross[v]) {
        if (!freeSlots.empty()) { crossSlot[v] = freeSlots.back(); freeSlots.pop_back(); }
        else crossSlot[v] = nCross++;
      }
      // a slot is released after its last consumer: that consumer's load precedes, in program order,
      // every store a later definition may make to the same slot
      for (int32_t c : dying[v]) freeSlots.push_back(crossSlot[c]);
    }
  }
  // tiles per group: 1 = each tile runs all chunks; more = each chunk runs on that many tiles in a row
  // (measured on a 53 k-node DAG: grouping is slower than streaming every chunk once per tile, so the
  // default stays 1)
  // (measured on the 53 k-node DAG with scope-local staging: 86.8 ms with one tile per chunk run, 96.0 with two,
  // 125.1 with four: every run reloads the table window, and the code is not what the kernel waits for)
  const int groupTiles = nChunks > 1 && opt.groupTiles > 0 ? opt.groupTiles : 1;
  const char* ldGlobal = lg ? "ld.global.f32" : "ld.global.f64";
  const char* stGlobal = lg ? "st.global.f32" : "st.global.f64";
  // ---- the DAG body: its own non-inlined function (the asm reads above must not move across the
  // barrier that follows the staging of a tile) ------------------------------------------------------
  std::vector<long long> winEnd(nChunks, 0);
  // operand ring (see emitBody): per chunk the operands it takes from earlier chunks, in the order of their first use
  std::vector<std::vector<int32_t>> ringOrderOf(pfSlots > 0 && nChunks > 1 ? nChunks : 0);
  for (size_t c = 0; c < ringOrderOf.size(); ++c) {
    std::vector<uint8_t> seen(n, 0);
    for (size_t v = chunkStart[c]; v < chunkStart[c + 1]; ++v)
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
        const int32_t ch = d.childIdx[e];
        if ((size_t)ch < chunkStart[c] && !seen[ch]) { seen[ch] = 1; ringOrderOf[c].push_back(ch); }
      }
  }
  // the first copies of a chunk are issued at the end of the chunk before it (they then overlap the staging of the
  // chunk's inputs), unless a chunk runs on several tiles in a row
  const bool ringAcross = groupTiles == 1;
  auto emitBody = [&](const std::string& fname, bool nanAware, size_t chunk) {
  const size_t v0 = chunkStart[chunk], v1 = chunkStart[chunk + 1];
  o << "static __device__ __noinline__ out_t " << fname << "(const unsigned xs_s, const unsigned cs_s, const unsigned tab_s, "
       "const unsigned lut_s, const real_t* __restrict__ tab_g, const unsigned char* __restrict__ lut_g, uint4* __restrict__ win, "
       "real_t* __restrict__ sc, const unsigned tid)\n{\n";
  o << "  const unsigned xs_t = xs_s + " << (asyncStage ? 4 * RS : rb) << "u * tid;\n  const unsigned cs_t = cs_s + " << cb << "u * tid;\n";
  if (asyncStage && NC > 0) {
    // codes of the discrete features, from this thread's raw row (unused ones are dropped by the compiler)
    for (int f = 0; f < F; ++f) {
      const FeatureMeta& fm = p.features[f];
      if (fm.codeSlot < 0) continue;
      o << "  int cf" << f << "; { unsigned raw; asm(\"ld.shared.b32 %0, [%1+" << 4 * f << "];\" : \"=r\"(raw) : \"r\"(xs_t));\n";
      if (floatIn) o << "    const float rf = __uint_as_float(raw); const unsigned rr = (unsigned)__float2int_rz(rf) - " << (unsigned)fm.lo << "u;\n";
      else if (p.ftype.kind == InKind::UInt) o << "    const unsigned rr = (raw > 2147483647u ? 2147483647u : raw) - " << (unsigned)fm.lo << "u;\n";
      else o << "    const unsigned rr = raw - " << (unsigned)fm.lo << "u;\n";
      o << "    cf" << f << " = rr < " << (unsigned)fm.domain << "u ? (int)rr + 2 : 1;";
      if (floatIn) o << " if (rf != rf) cf" << f << " = 0;";
      o << " }\n";
    }
  }
  // both variants of a chunk leave the same table window behind; a variant that skips a chunk (no staged
  // values: nothing NaN-sensitive in it) continues from what the plain body of that chunk leaves
  winBase = chunk == 0 ? 0 : winEnd[chunk - 1];
  // with grouped tiles a chunk runs several times in a row: it cannot rely on the window its predecessor left
  if (streamed && (chunk == 0 || groupTiles > 1)) swapWindow(o, winBase);
  std::vector<uint8_t> loaded(nChunks > 1 ? n : 0, 0);
  std::vector<std::string> terms;
  if (scoped && nChunks > 1 && pfSlots == 0) {
    // Operands defined by earlier chunks: when they are few, all of them are requested at the top of the
    // function, so that their latencies (L2 or DRAM) overlap instead of standing in front of every first use.
    // (Not together with the operand ring, which accounts for every operand of an earlier chunk itself.)
    std::vector<int32_t> incoming;
    for (size_t v = v0; v < v1; ++v)
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
        const int32_t c = d.childIdx[e];
        if ((size_t)c < v0 && !loaded[c]) { loaded[c] = 1; incoming.push_back(c); }
      }
    if (incoming.size() <= (size_t)std::max(opt.hoistLoads, 0)) {
      for (int32_t c : incoming)
        o << "  real_t " << V(c) << "; asm volatile(\"" << ldGlobal << " %0, [%1+" << (long long)crossSlot[c] * TILE * rb
          << "];\" : \"=" << cReal << "\"(" << V(c) << ") : \"l\"(sc) : \"memory\");\n";
    } else {
      for (int32_t c : incoming) loaded[c] = 0;
    }
  }
  // Operands defined by an earlier chunk are fetched from the scratch area `loadAhead` nodes before the node
  // that uses them first (0: at the first use): the request is then in flight while the nodes in between are
  // evaluated, at the price of one register per outstanding value.  Moving such a load up crosses no store to
  // its slot: a slot is released only after its value's last consumer, and that consumer is not before the
  // node the load was moved up from, so no node in between can have been given the slot.
  // Operand ring (scope-local staging, prefetchSlots > 0): the operands a chunk takes from earlier chunks are
  // copied scratch -> shared memory with cp.async, in the order of their first use, `prefetchSlots` of them ahead
  // of the evaluation; a use waits for its own copy group (the groups complete in order), reads its slot and
  // hands the slot to the next copy.  Thread = sample on both sides, so no barrier is involved, the copies hold
  // no registers, and the assembler cannot move them back down to the uses.
  std::vector<int32_t> ringIndex(pfSlots > 0 && nChunks > 1 ? n : 0, -1);   // per incoming operand: its place in the order
  const std::vector<int32_t> noOrder;
  const std::vector<int32_t>& ringOrder = ringIndex.empty() ? noOrder : ringOrderOf[chunk];
  size_t ringIssued = 0;
  auto ringCopy = [&](const std::vector<int32_t>& order, size_t k) {
    o << "  asm volatile(\"cp.async.ca.shared.global [%0+" << (k % (size_t)pfSlots) * TILE * 4 << "], [%1+"
      << (long long)crossSlot[order[k]] * TILE * rb << "], 4; cp.async.commit_group;\" :: \"r\"(pf_t), \"l\"(sc) : \"memory\");\n";
  };
  if (!ringIndex.empty()) {
    for (size_t k = 0; k < ringOrder.size(); ++k) ringIndex[ringOrder[k]] = (int32_t)k;
    o << "  const unsigned pf_t = xs_s + " << offPf << "u + 4u * tid;\n";
    const size_t first = std::min(ringOrder.size(), (size_t)pfSlots);
    if (ringAcross && chunk > 0) ringIssued = first;   // in flight since the end of the chunk before
    else while (ringIssued < first) ringCopy(ringOrder, ringIssued++);
  }
  const size_t loadAhead = nChunks > 1 && ringIndex.empty() ? (size_t)std::max(opt.loadAhead, 0) : 0;
  // loadMode 1: the early request is a prefetch into L1 (no register is held), the load stays at the first use;
  // loadMode 2: the early load is a volatile one, which the assembler does not move back down to its use
  const int loadMode = opt.loadMode;
  const char* ldEarly = loadMode == 2 ? (lg ? "ld.volatile.global.f32" : "ld.volatile.global.f64") : ldGlobal;
  std::vector<uint8_t> requested(nChunks > 1 ? n : 0, 0);
  size_t aheadDone = v0;   // nodes [v0, aheadDone) have had their operands requested
  auto emitLoad = [&](int32_t c, const char* op) {
    loaded[c] = 1;
    o << "  real_t " << V(c) << "; asm volatile(\"" << op << " %0, [%1+" << (long long)crossSlot[c] * TILE * rb
      << "];\" : \"=" << cReal << "\"(" << V(c) << ") : \"l\"(sc) : \"memory\");\n";
  };
  for (size_t v = v0; v < v1; ++v) {
    if (nChunks > 1) {
      const size_t upTo = std::min(v1, v + loadAhead + 1);
      for (size_t u = std::max(aheadDone, v); u < upTo && ringIndex.empty(); ++u)
        for (int64_t e = d.childPtr[u]; e < d.childPtr[u + 1]; ++e) {
          const int32_t c = d.childIdx[e];
          if ((size_t)c >= v0 || loaded[c] || requested[c]) continue;
          requested[c] = 1;
          if (loadMode == 1 && u > v)
            o << "  asm volatile(\"prefetch.global.L1 [%0+" << (long long)crossSlot[c] * TILE * rb << "];\" :: \"l\"(sc) : \"memory\");\n";
          else
            emitLoad(c, u > v ? ldEarly : ldGlobal);
        }
      aheadDone = std::max(aheadDone, upTo);
      for (int64_t e = d.childPtr[v]; e < d.childPtr[v + 1]; ++e) {
        const int32_t c = d.childIdx[e];
        if ((size_t)c >= v0 || loaded[c]) continue;
        if (ringIndex.empty()) { emitLoad(c, ldGlobal); continue; }
        // groups newer than this operand's may still be pending
        const size_t k = (size_t)ringIndex[c];
        loaded[c] = 1;
        o << "  real_t " << V(c) << "; asm volatile(\"cp.async.wait_group " << (ringIssued - 1 - k) << "; ld.shared.f32 %0, [%1+"
          << (k % (size_t)pfSlots) * TILE * 4 << "];\" : \"=f\"(" << V(c) << ") : \"r\"(pf_t) : \"memory\");\n";
        if (ringIssued < ringOrder.size()) ringCopy(ringOrder, ringIssued++);
      }
    }
    if (opt.syncEvery > 0 && v > 0 && v % (size_t)opt.syncEvery == 0) o << "  __syncthreads();\n";
    const std::string name = V((int32_t)v);
    int64_t lo = d.childPtr[v], hi = d.childPtr[v + 1];
    switch (d.kind[v]) {
      case kGaussian: {
        double sd = d.stddev[v];
        std::string x = "x" + std::to_string(v);
        o << readX(x, scoped ? leafSlot[v] : (asyncStage ? d.feature[v] : p.features[d.feature[v]].valueSlot), (long long)v);
        if (lg) {
          float mu = (float)d.mean[v];
          float c2 = (float)(-(1.0 / (2.0 * sd * sd)) * LOG2E);
          float c1 = (float)((-std::log(sd) - 0.5 * std::log(2 * M_PI)) * LOG2E);
          o << "  const float d" << v << " = " << x << " - " << lit32(mu) << ";\n";
          if (opt.gaussForm == 1) {
            // c2 * (d*d + c1/c2): one add, one fma whose addend is a constant, one multiply
            o << "  " << (nanAware ? "float " : "const float ") << name << " = fmaf(d" << v << ", d" << v << ", " << lit32((float)((double)c1 / (double)c2)) << ") * " << lit32(c2) << ";\n";
          } else {
            o << "  " << (nanAware ? "float " : "const float ") << name << " = fmaf(d" << v << " * d" << v << ", " << lit32(c2) << ", " << lit32(c1) << ");\n";
          }
          if (nanAware) o << "  " << name << " = (d" << v << " != d" << v << ") ? 0.0f : " << name << ";\n";
        } else {
          double var = sd * sd;
          double coef = 1.0 / std::sqrt(2.0 * M_PI * var);
          double den = -1.0 / (2.0 * var);
          o << "  const double d" << v << " = " << x << " - " << lit64(d.mean[v]) << ";\n";
          o << "  " << (nanAware ? "double " : "const double ") << name << " = " << lit64(coef) << " * exp((d" << v << " * d" << v << ") * " << lit64(den) << ");\n";
          if (nanAware) o << "  " << name << " = (d" << v << " != d" << v << ") ? 1.0 : " << name << ";\n";
        }
        break;
      }
      case kCategorical:
      case kHistogram:
        if (fusedAway[v]) break;   // read by its group's first leaf
        if (fusedHead[v] >= 0) {
          // combined code of the group's leaves, then one read of the fused table
          const FusedGroup& g = fused[(size_t)fusedHead[v]];
          std::string idx;
          for (size_t q = g.leaves.size(); q-- > 0;) {
            const int32_t c = g.leaves[q];
            const FeatureMeta& fm = p.features[p.groups[d.group[c]].feature];
            const std::string cn = "c" + std::to_string(c);
            o << readCode(cn, fm.codeSlot, (long long)c);
            idx = idx.empty() ? cn : "(" + cn + " + " + std::to_string(fm.domain + 2) + " * " + idx + ")";
          }
          o << "  const int fi" << v << " = " << idx << ";\n";
          o << readTab(name, g.offset, "fi" + std::to_string(v), (long long)v);
          break;
        }
        if (streamed && (p.tabOffset[v] + tableEntriesOf(v) - winBase) * rb > (long long)winBytes) swapWindow(o, p.tabOffset[v]);
        emitLeafLookup(o, v, name);
        break;
      case kProduct: {
        terms.clear();
        for (int64_t e = lo; e < hi; ++e)
          if (!fusedAway[d.childIdx[e]]) terms.push_back(V(d.childIdx[e]));
        const char* op = lg ? " + " : " * ";
        o << "  const real_t " << name << " = "
          << balanced(terms, 0, terms.size(), [&](const std::string& a, const std::string& b) { return "(" + a + op + b + ")"; }) << ";\n";
        break;
      }
      default: {
        const int64_t k = hi - lo;
        if (!lg) {
          terms.clear();
          for (int64_t e = lo; e < hi; ++e) terms.push_back("(" + lit64(d.weight[e]) + " * " + V(d.childIdx[e]) + ")");
          o << "  const double " << name << " = "
            << balanced(terms, 0, terms.size(), [&](const std::string& a, const std::string& b) { return "(" + a + " + " + b + ")"; }) << ";\n";
          break;
        }
        if (k == 1) {
          float w = (float)std::log2(d.weight[lo]);
          if (w == 0.0f) o << "  const float " << name << " = " << V(d.childIdx[lo]) << ";\n";
          else o << "  const float " << name << " = " << V(d.childIdx[lo]) << " + " << lit32(w) << ";\n";
          break;
        }
        terms.clear();
        for (int64_t e = lo; e < hi; ++e) {
          std::string t = "t" + std::to_string(v) + "_" + std::to_string(e - lo);
          o << "  const float " << t << " = " << V(d.childIdx[e]) << " + " << lit32((float)std::log2(d.weight[e])) << ";\n";
          terms.push_back(t);
        }
        if (opt.useMax3) o << "  const float m" << v << " = " << max3Tree(terms, 0, terms.size()) << ";\n";
        else o << "  const float m" << v << " = "
               << balanced(terms, 0, terms.size(), [&](const std::string& a, const std::string& b) { return "fmaxf(" + a + ", " + b + ")"; }) << ";\n";
        std::string mm = "m" + std::to_string(v);
        if (mayNeg[v]) {
          o << "  const float mm" << v << " = (m" << v << " == NEG_INF) ? 0.0f : m" << v << ";\n";
          mm = "mm" + std::to_string(v);
        }
        for (auto& t : terms) t = "ex2(" + t + " - " + mm + ")";
        o << "  const float s" << v << " = "
          << balanced(terms, 0, terms.size(), [&](const std::string& a, const std::string& b) { return "(" + a + " + " + b + ")"; }) << ";\n";
        o << "  const float " << name << " = m" << v << " + lg2(s" << v << ");\n";
      }
    }
    if (crossSlot[v] >= 0)
      o << "  asm volatile(\"" << stGlobal << " [%0+" << (long long)crossSlot[v] * TILE * rb << "], %1;\" :: \"l\"(sc), \""
        << cReal << "\"(" << name << ") : \"memory\");\n";
  }
  if (!ringIndex.empty() && ringAcross && chunk + 1 < nChunks) {
    const std::vector<int32_t>& next = ringOrderOf[chunk + 1];
    for (size_t k = 0; k < next.size() && k < (size_t)pfSlots; ++k) ringCopy(next, k);
  }
  if (v1 < n) o << "  return (out_t)0;\n}\n";
  else if (lg) o << "  return " << V(d.root()) << " * 0x1.62e43p-1f;\n}\n";  // log2 -> ln
  else o << "  return log(" << V(d.root()) << ");\n}\n";
  winEnd[chunk] = winBase;

  };
  for (int variant = 0; variant < (twoBodies ? 2 : 1); ++variant)
    for (size_t c = 0; c < nChunks; ++c) {
      if (scoped && variant == 1 && chunkValueFeat[c].empty()) continue;
      emitBody(std::string(variant ? "spnb_body_nan" : "spnb_body") + std::to_string(c),
               twoBodies ? variant == 1 : (p.marginal && floatIn), c);
    }

  if (scoped) {
    // ---- kernel, scope-local staging: per tile, every chunk stages its own features from the feature-major
    // copy (thread = sample: coalesced global reads, conflict-free shared writes, no transposition) --------
    // CF: per chunk its value features, then (feature, lo, domain) per code feature
    std::vector<size_t> cfOff(nChunks);
    o << "__device__ const int CF[] = {";
    size_t cfN = 0;
    for (size_t c = 0; c < nChunks; ++c) {
      cfOff[c] = cfN;
      for (int32_t f : chunkValueFeat[c]) { o << (cfN ? "," : "") << f; ++cfN; }
      // (domain stored as -domain - 1: the feature's special codes are the clamped ones)
      for (int32_t f : chunkCodeFeat[c]) {
        const FeatureMeta& fm = p.features[f];
        if (codePlane) { o << (cfN ? "," : "") << fm.codeSlot; ++cfN; continue; }   // its row of the code plane
        o << (cfN ? "," : "") << f << "," << fm.lo << "," << (clampAllowed && fm.clampCodes ? -fm.domain - 1 : fm.domain);
        cfN += 3;
      }
    }
    if (!cfN) o << "0";
    o << "};\n";
    // One staging routine for all chunks, out of line: the kernel below stays a short list of calls (the
    // JIT's time grows quadratically with the memory operations it sees in one function).
    o << "typedef " << (cb == 1 ? "unsigned char" : "unsigned short") << " code_t;\n";
    o << "static __device__ __noinline__ int spnb_stage(unsigned char* __restrict__ smem, const float* __restrict__ src, const code_t* __restrict__ srcc, const unsigned long long ld,\n"
         "                                              const int* __restrict__ cf, const int nv, const int nc, const unsigned codeBase, const unsigned tid)\n{\n";
    o << "  float* xs = reinterpret_cast<float*>(smem);\n  code_t* cs = reinterpret_cast<code_t*>(smem + codeBase);\n  int nan = 0;\n";
    o << "#pragma unroll " << std::max(opt.stageUnroll, 1) << "\n";
    o << "  for (int j = 0; j < nv; ++j) { const float raw = src[(unsigned long long)__ldg(cf + j) * ld]; xs[j * SX + tid] = raw; nan |= (raw != raw); }\n";
    o << "  cf += nv;\n";
    o << "#pragma unroll " << std::max(opt.stageUnroll, 1) << "\n";
    if (codePlane) {
      // the codes were made with the feature-major copy: one byte (half-word) per sample and feature
      o << "  for (int j = 0; j < nc; ++j) cs[j * SX + tid] = srcc[(unsigned long long)__ldg(cf + j) * ld];\n";
      o << "  return nan;\n}\n";
    } else {
    o << "  for (int j = 0; j < nc; ++j) {\n";
    o << "    const float raw = src[(unsigned long long)__ldg(cf + 3 * j) * ld];\n";
    o << "    const unsigned rr = (unsigned)TOINT(raw) - (unsigned)__ldg(cf + 3 * j + 1);\n";
    o << "    const int dm = __ldg(cf + 3 * j + 2);\n";
    o << "    const bool cl = dm < 0;\n";
    o << "    const int dom = cl ? -dm - 1 : dm;\n";
    o << "    int code = rr < (unsigned)dom ? (int)rr + 2 : (cl ? dom + 2 : 1);\n";
    o << "    if (raw != raw) code = cl ? 65535 : 0;\n";
    o << "    cs[j * SX + tid] = (code_t)code;\n";
    o << "  }\n  return nan;\n}\n";
    }
    o << "extern \"C\" __global__ void __launch_bounds__(TILE, 1)\n";
    o << "spnb_kernel(const float* __restrict__ xt, out_t* __restrict__ out, unsigned long long n, const real_t* __restrict__ tab_g, const unsigned char* __restrict__ lut_g, real_t* __restrict__ scratch, unsigned long long ld)\n{\n";
    if (nCross > 0) o << "  real_t* sc = scratch + ((size_t)blockIdx.x * " << (size_t)nCross * (size_t)groupTiles << "u * TILE + threadIdx.x);\n";
    else o << "  real_t* sc = scratch;\n";
    o << "  extern __shared__ __align__(16) unsigned char smem_raw[];\n";
    o << "  const unsigned tid = threadIdx.x;\n";
    o << "  const unsigned xs_s = (unsigned)__cvta_generic_to_shared(smem_raw);\n";
    o << "  unsigned tab_s = 0, lut_s = 0;\n";
    o << "  uint4* win = reinterpret_cast<uint4*>(smem_raw + " << offTab << ");\n";
    if (tabSmem) {
      o << "  tab_s = (unsigned)__cvta_generic_to_shared(win);\n";
      if (!streamed) o << "  for (unsigned i = tid; i < NTAB; i += TILE) reinterpret_cast<real_t*>(win)[i] = tab_g[i];\n";
    }
    if (lutSmem) {
      o << "  { unsigned char* lut = smem_raw + " << offLut << ";\n";
      o << "    for (unsigned i = tid; i < NLUT; i += TILE) lut[i] = lut_g[i];\n    lut_s = (unsigned)__cvta_generic_to_shared(lut); }\n";
    }
    if ((tabSmem && !streamed) || lutSmem) o << "  __syncthreads();   // tables loaded above are read by every thread\n";
    o << "  const unsigned long long ntiles = (n + TILE - 1) / TILE;\n";
    // Every chunk runs on groupTiles tiles in a row (each with its own slice of the cross-chunk scratch), so
    // that its code, which fits the instruction cache, is fetched once per group instead of once per tile.
    // (a batch with fewer tiles than that per CTA is cut into smaller groups, so that every CTA gets work)
    o << "  unsigned G = (unsigned)(ntiles / gridDim.x);\n";
    o << "  G = G < 1u ? 1u : (G > " << groupTiles << "u ? " << groupTiles << "u : G);\n";
    o << "  const unsigned long long ngroups = (ntiles + G - 1) / G;\n";
    o << "#pragma unroll 1\n";
    o << "  for (unsigned long long group = blockIdx.x; group < ngroups; group += gridDim.x) {\n";
    for (size_t c = 0; c < nChunks; ++c) {
      const size_t nv = chunkValueFeat[c].size(), nc = chunkCodeFeat[c].size();
      o << "    // chunk " << c << ": " << nv << " staged values, " << nc << " staged codes\n";
      o << "#pragma unroll 1\n";
      o << "    for (unsigned t = 0; t < G; ++t) {\n";
      o << "      const unsigned long long tile = group * G + t;\n";
      o << "      if (tile >= ntiles) break;\n";
      o << "      const unsigned long long base = tile * TILE;\n";
      o << "      const unsigned rows = (n - base) < (unsigned long long)TILE ? (unsigned)(n - base) : (unsigned)TILE;\n";
      o << "      // threads past the end of the batch repeat its last sample; their result is not stored\n";
      o << "      const float* __restrict__ src = xt + base + (tid < rows ? tid : rows - 1);\n";
      o << "      const code_t* __restrict__ srcc = reinterpret_cast<const code_t*>(xt + (unsigned long long)NF * ld) + base + (tid < rows ? tid : rows - 1);\n";
      o << "      real_t* sct = sc + (size_t)t * " << nCross << "u * TILE;\n";
      // Thread = sample on both sides of the staging area: a thread stages and reads its own column only, so
      // the chunks need no CTA-wide barrier between them.  Without one the warps drift apart and one warp's
      // staging loads overlap the other warps' arithmetic; the plain / NaN-aware choice is then made per warp.
      // (The barriers around a swap of the table window stay: every warp passes the same swaps in the same
      // order, whichever variants it takes.)
      const bool barrier = opt.chunkBarrier != 0;
      const std::string anyNan = barrier ? "__syncthreads_or(nan)" : "__any_sync(0xffffffffu, nan)";
      if (barrier) o << "      __syncthreads();\n";
      const bool choose = twoBodies && nv > 0;
      o << "      " << (choose ? "const int nan = " : "") << "spnb_stage(smem_raw, src, srcc, ld, CF + " << cfOff[c] << ", " << nv << ", " << nc << ", "
        << codeBase(c) << "u, tid);\n";
      const std::string args = "(xs_s, xs_s + " + std::to_string(codeBase(c)) + "u, tab_s, lut_s, tab_g, lut_g, win, sct, tid);\n";
      const bool last = c + 1 == nChunks;
      const std::string lhs = last ? "const out_t res = " : "";
      if (choose) {
        if (last) {
          o << "      out_t res;\n";
          o << "      if (" << anyNan << ") res = spnb_body_nan" << c << args;
          o << "      else res = spnb_body" << c << args;
        } else {
          o << "      if (" << anyNan << ") spnb_body_nan" << c << args;
          o << "      else spnb_body" << c << args;
        }
      } else {
        if (barrier) o << "      __syncthreads();\n";
        o << "      " << lhs << "spnb_body" << c << args;
      }
      if (last) o << "      if (tid < rows) out[base + tid] = res;\n";
      o << "    }\n";
    }
    o << "  }\n}\n";
    if (info) {
      info->kernelName = "spnb_kernel";
      info->tile = TILE;
      info->inputStride = SX;
      info->tablesInSmem = tabSmem;
      info->tableEntries = tabEntries;
      info->fusedTable = fusedTable;
      info->fusedGroups = (int)fused.size();
      info->dynamicSmemBytes = smemTotal;
      info->scratchSlots = nCross * groupTiles;
      info->scoped = true;
      info->codePlaneBytes = codePlane ? cb : 0;
      info->numChunks = (int)nChunks;
    }
    return o.str();
  }

  if (asyncStage) {
    // ---- kernel, asynchronous staging: the next tile travels into the other buffer while this one is
    // evaluated; rows are stored in order with stride RS words ---------------------------------------------
    o << "#define RS " << RS << "\n";
    o << "extern \"C\" __global__ void __launch_bounds__(TILE, " << minBlocks << ")\n";
    o << "spnb_kernel(const in_t* __restrict__ in, out_t* __restrict__ out, unsigned long long n, const real_t* __restrict__ tab_g, const unsigned char* __restrict__ lut_g, real_t* __restrict__ scratch)\n{\n";
    if (nCross > 0) o << "  real_t* sc = scratch + ((size_t)blockIdx.x * " << (size_t)nCross << "u * TILE + threadIdx.x);\n";
    else o << "  real_t* sc = scratch;\n";
    o << "  extern __shared__ __align__(16) unsigned char smem_raw[];\n";
    o << "  const unsigned tid = threadIdx.x;\n";
    o << "  const unsigned buf_s = (unsigned)__cvta_generic_to_shared(smem_raw);\n";
    o << "  uint4* win = reinterpret_cast<uint4*>(smem_raw + " << offTab << ");\n";
    o << "  unsigned tab_s = 0, lut_s = 0;\n";
    // Every CTA takes one contiguous range of rows (whole warps), in tiles of TILE rows, the last one partial: a
    // batch of a few tiles per CTA then costs what its rows cost instead of a whole number of tile rounds (warps
    // past the end of the range skip the body, which has no barrier in it).
    o << "  const unsigned long long per = ((n + gridDim.x - 1) / gridDim.x + 31ull) & ~31ull;\n";
    o << "  const unsigned long long lo = (unsigned long long)blockIdx.x * per;\n";
    o << "  const unsigned long long hi = lo + per < n ? lo + per : n;\n";
    o << "  // copy of one tile: element e of the tile's row-major block goes to word (e / NF) * RS + e % NF\n";
    o << "  auto issue = [&](unsigned long long base, unsigned buf) {\n";
    o << "    const unsigned rows = (hi - base) < (unsigned long long)TILE ? (unsigned)(hi - base) : (unsigned)TILE;\n";
    o << "    const in_t* __restrict__ src = in + base * NF;\n";
    o << "    const unsigned total = rows * NF;\n";
    o << "    const unsigned dst = buf_s + buf * " << asyncBuf << "u;\n";
    o << "#pragma unroll 4\n";
    o << "    for (unsigned e = tid; e < total; e += TILE) {\n";
    o << "      const unsigned r = e / NF;\n";
    o << "      asm volatile(\"cp.async.ca.shared.global [%0], [%1], 4;\" :: \"r\"(dst + 4u * (e + r * (RS - NF))), \"l\"(src + e) : \"memory\");\n";
    o << "    }\n";
    o << "    asm volatile(\"cp.async.commit_group;\" ::: \"memory\");\n";
    o << "  };\n";
    o << "  if (lo < hi) issue(lo, 0u);\n";
    // (the tables are fetched while the first tile's copies are in flight)
    if (tabSmem) {
      // resident leaf tables behind the two buffers; the first barrier of the tile loop orders them before any read
      o << "  tab_s = (unsigned)__cvta_generic_to_shared(win);\n";
      o << "  for (unsigned i = tid; i < NTAB; i += TILE) reinterpret_cast<real_t*>(win)[i] = tab_g[i];\n";
    }
    if (lutSmem) {
      o << "  { unsigned char* lut = smem_raw + " << offLut << ";\n";
      o << "    for (unsigned i = tid; i < NLUT; i += TILE) lut[i] = lut_g[i];\n    lut_s = (unsigned)__cvta_generic_to_shared(lut); }\n";
    }
    o << "  unsigned cur = 0;\n";
    o << "#pragma unroll 1\n";
    o << "  for (unsigned long long base = lo; base < hi; base += TILE) {\n";
    o << "    const unsigned rows = (hi - base) < (unsigned long long)TILE ? (unsigned)(hi - base) : (unsigned)TILE;\n";
    o << "    asm volatile(\"cp.async.wait_group 0;\" ::: \"memory\");\n";
    o << "    __syncthreads();   // this tile has landed for every thread; the other buffer's readers are done\n";
    o << "    if (base + TILE < hi) issue(base + TILE, cur ^ 1u);\n";
    o << "    const unsigned xs_s = buf_s + cur * " << asyncBuf << "u;\n";
    o << "    out_t res = (out_t)0;\n";
    // the bodies hold no barrier (tables are resident) unless one was asked for
    o << "    const bool active = " << (opt.syncEvery > 0 ? "true" : "(tid & ~31u) < rows") << ";\n";
    auto chainA = [&](const char* prefix, const std::string& in2) {
      o << in2 << "if (active) {\n";
      for (size_t c = 0; c < nChunks; ++c)
        o << in2 << "  " << (c + 1 == nChunks ? "res = " : "") << prefix << c << "(xs_s, 0u, tab_s, lut_s, tab_g, lut_g, win, sc, tid);\n";
      o << in2 << "}\n";
    };
    if (twoBodies) {
      o << "    int nan = 0;\n";
      o << "    if (tid < rows) {\n      const float* row = reinterpret_cast<const float*>(smem_raw + cur * " << asyncBuf << "u) + tid * RS;\n";
      o << "#pragma unroll\n      for (int c = 0; c < NF; ++c) nan |= (row[c] != row[c]);\n    }\n";
      o << "    if (__syncthreads_or(nan)) {\n";
      chainA("spnb_body_nan", "      ");
      o << "    } else {\n";
      chainA("spnb_body", "      ");
      o << "    }\n";
    } else {
      chainA("spnb_body", "    ");
    }
    o << "    if (tid < rows) out[base + tid] = res;\n";
    o << "    cur ^= 1u;\n";
    o << "  }\n}\n";
    if (info) {
      info->kernelName = "spnb_kernel";
      info->tile = TILE;
      info->inputStride = RS;
      info->tablesInSmem = tabSmem;
      info->tableEntries = tabEntries;
      info->fusedTable = fusedTable;
      info->fusedGroups = (int)fused.size();
      info->dynamicSmemBytes = smemTotal;
      info->scratchSlots = nCross;
      info->scoped = false;
      info->numChunks = (int)nChunks;
    }
    return o.str();
  }

  // ---- kernel: persistent CTAs, stage a tile of TILE samples, evaluate, store -------------------
  o << "extern \"C\" __global__ void __launch_bounds__(TILE, " << minBlocks << ")\n";
  o << "spnb_kernel(const in_t* __restrict__ in, out_t* __restrict__ out, unsigned long long n, const real_t* __restrict__ tab_g, const unsigned char* __restrict__ lut_g, real_t* __restrict__ scratch)\n{\n";
  if (nCross > 0) o << "  real_t* sc = scratch + ((size_t)blockIdx.x * " << (size_t)nCross * (size_t)std::max(groupTiles, 1) << "u * TILE + threadIdx.x);\n";
  else o << "  real_t* sc = scratch;\n";
  o << "  extern __shared__ __align__(16) unsigned char smem_raw[];\n";
  o << "  const unsigned tid = threadIdx.x;\n";
  o << "  real_t* xs = reinterpret_cast<real_t*>(smem_raw + " << offXs << ");\n";
  o << "  typedef " << (cb == 1 ? "unsigned char" : "unsigned short") << " code_t;\n";
  o << "  code_t* cs = reinterpret_cast<code_t*>(smem_raw + " << offCs << ");\n";
  o << "  const unsigned xs_s = (unsigned)__cvta_generic_to_shared(xs);\n  const unsigned cs_s = (unsigned)__cvta_generic_to_shared(cs);\n";
  o << "  unsigned tab_s = 0, lut_s = 0;\n";
  if (twoBodies) o << "  int* nanrow = reinterpret_cast<int*>(smem_raw + " << offNan << ");\n  nanrow[tid] = 0;\n";
  if (!identity) {
    o << "  int4* fm = reinterpret_cast<int4*>(smem_raw + " << offFm << ");\n";
    o << "  for (unsigned i = tid; i < NF; i += TILE) fm[i] = make_int4(FM[4 * i], FM[4 * i + 1], FM[4 * i + 2], FM[4 * i + 3]);\n";
  }
  o << "  uint4* win = reinterpret_cast<uint4*>(smem_raw + " << offTab << ");\n";
  if (tabSmem) {
    o << "  tab_s = (unsigned)__cvta_generic_to_shared(win);\n";
    if (!streamed) o << "  for (unsigned i = tid; i < NTAB; i += TILE) reinterpret_cast<real_t*>(win)[i] = tab_g[i];\n";
  }
  if (lutSmem) {
    o << "  { unsigned char* lut = smem_raw + " << offLut << ";\n";
    o << "    for (unsigned i = tid; i < NLUT; i += TILE) lut[i] = lut_g[i];\n    lut_s = (unsigned)__cvta_generic_to_shared(lut); }\n";
  }
  o << "  const unsigned long long ntiles = (n + TILE - 1) / TILE;\n";
  // staging of one tile: coalesced reads of TILE x NF inputs, transposed (and digested) into shared memory
  auto emitStage = [&](const std::string& ind) {
    o << ind << "const unsigned long long base = tile * TILE;\n";
    o << ind << "const unsigned rows = (n - base) < (unsigned long long)TILE ? (unsigned)(n - base) : (unsigned)TILE;\n";
    o << ind << "__syncthreads();\n";
    o << ind << "{\n";
    o << ind << "  const in_t* __restrict__ src = in + base * NF;\n";
    o << ind << "  const unsigned total = rows * NF;\n";
    if (identity) {
      o << "#pragma unroll " << std::max(opt.rowStageUnroll, 1) << "\n";
      o << ind << "  for (unsigned e = tid; e < total; e += TILE) { const unsigned r = e / NF; const unsigned c = e - r * NF; const in_t raw = src[e]; xs[c * SX + r] = (real_t)raw;" << (twoBodies ? " if (raw != raw) nanrow[r] = 1;" : "") << " }\n";
      o << ind << "  if (rows < TILE) for (unsigned e = total + tid; e < TILE * NF; e += TILE) { const unsigned r = e / NF; const unsigned c = e - r * NF; xs[c * SX + r] = (real_t)0; }\n";
    } else {
      o << "#pragma unroll " << std::max(opt.rowStageUnroll, 1) << "\n";
      o << ind << "  for (unsigned e = tid; e < TILE * NF; e += TILE) {\n";
      o << ind << "    const unsigned r = e / NF; const unsigned c = e - r * NF;\n";
      o << ind << "    const int4 m = fm[c];\n";
      o << ind << "    const bool live = e < total;\n";
      o << ind << "    in_t raw = 0; if (live) raw = src[e];\n";
      if (NV) o << ind << "    if (m.w >= 0) { xs[m.w * SX + r] = (real_t)raw;" << (twoBodies ? " if (raw != raw) nanrow[r] = 1;" : "") << " }\n";
      if (NC) {
        o << ind << "    if (m.z >= 0) {\n";
        o << ind << "      const unsigned rr = (unsigned)TOINT(raw) - (unsigned)m.x;\n";
        if (anyClamp) {
          o << ind << "      const bool cl = m.z >= 65536;\n";
          o << ind << "      const int oor = cl ? m.y + 2 : 1;\n";
          o << ind << "      int code = rr < (unsigned)m.y ? (int)rr + 2 : oor;\n";
          if (floatIn) o << ind << "      if (raw != raw) code = cl ? 65535 : 0;\n";
          o << ind << "      cs[(m.z & 65535) * SX + r] = (code_t)(live ? code : oor);\n";
        } else {
          o << ind << "      int code = rr < (unsigned)m.y ? (int)rr + 2 : 1;\n";
          if (floatIn) o << ind << "      if (raw != raw) code = 0;\n";
          o << ind << "      cs[m.z * SX + r] = (code_t)(live ? code : 1);\n";
        }
        o << ind << "    }\n";
      }
      o << ind << "  }\n";
    }
    o << ind << "}\n";
    o << ind << "__syncthreads();\n";
  };
  // call of chunks [c0, c1) on the staged tile; the plain / NaN-aware choice is uniform over the CTA, so
  // barriers inside the bodies stay legal
  auto emitCalls = [&](const std::string& ind, size_t c0, size_t c1, const char* scratchPtr) {
    auto chain = [&](const char* prefix, const std::string& in2) {
      for (size_t c = c0; c < c1; ++c)
        o << in2 << (c + 1 == nChunks ? "res = " : "") << prefix << c << "(xs_s, cs_s, tab_s, lut_s, tab_g, lut_g, win, "
          << scratchPtr << ", tid);\n";
    };
    if (twoBodies) {
      o << ind << "const int mynan = nanrow[tid];\n" << ind << "nanrow[tid] = 0;\n";
      o << ind << "if (__syncthreads_or(mynan)) {\n";
      chain("spnb_body_nan", ind + "  ");
      o << ind << "} else {\n";
      chain("spnb_body", ind + "  ");
      o << ind << "}\n";
    } else {
      chain("spnb_body", ind);
    }
  };
  if (groupTiles <= 1) {
    o << "#pragma unroll 1\n";
    o << "  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {\n";
    emitStage("    ");
    o << "    out_t res;\n";
    emitCalls("    ", 0, nChunks, "sc");
    o << "    if (tid < rows) out[base + tid] = res;\n";
    o << "  }\n}\n";
  } else {
    // A chunk's code stays in the instruction caches while it runs on groupTiles tiles in a row; every
    // (chunk, tile) pair stages the tile again (it is still in L2) and keeps its own scratch slice.
    o << "  const unsigned long long ngroups = (ntiles + " << groupTiles << " - 1) / " << groupTiles << ";\n";
    o << "#pragma unroll 1\n";
    o << "  for (unsigned long long group = blockIdx.x; group < ngroups; group += gridDim.x) {\n";
    for (size_t c = 0; c < nChunks; ++c) {
      o << "#pragma unroll 1\n";
      o << "    for (unsigned t = 0; t < " << groupTiles << "u; ++t) {\n";
      o << "      const unsigned long long tile = group * " << groupTiles << " + t;\n";
      o << "      if (tile >= ntiles) break;\n";
      emitStage("      ");
      o << "      real_t* sct = sc + (size_t)t * " << nCross << "u * TILE;\n";
      o << "      out_t res = (out_t)0;\n";
      emitCalls("      ", c, c + 1, "sct");
      if (c + 1 == nChunks) o << "      if (tid < rows) out[base + tid] = res;\n";
      o << "    }\n";
    }
    o << "  }\n}\n";
  }

  if (info) {
    info->kernelName = "spnb_kernel";
    info->tile = TILE;
    info->inputStride = SX;
    info->tablesInSmem = tabSmem;
    info->tableEntries = tabEntries;
      info->fusedTable = fusedTable;
      info->fusedGroups = (int)fused.size();
    info->dynamicSmemBytes = smemTotal;
    info->scratchSlots = nCross * std::max(groupTiles, 1);
    info->scoped = false;
    info->numChunks = (int)nChunks;
  }
  return o.str();
}

}  // namespace spnb
