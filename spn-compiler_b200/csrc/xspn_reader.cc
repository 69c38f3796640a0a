// Native reader of xspn files: a small, bounds-checked Cap'n Proto decoder specialised to the
// reference's schema (xspn/xspn/serialization/binary/capnproto/spflow.capnp:27-101).
// Supports the unpacked stream framing with any number of segments, struct / list / far /
// double-far pointers, inline-composite lists and structs shorter than the schema (missing
// fields read as zero).  Semantics of what is read follow the reference's front end
// (compiler/src/pipeline/steps/frontend/SPFlowToMLIRDeserializer.cpp:63-258).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <regex>
#include <unordered_map>

#include "model.h"

namespace spnb {

namespace {

[[noreturn]] void fail(const std::string& msg) { throw std::runtime_error(msg); }

struct Message {
  const uint8_t* data;
  size_t size;
  std::vector<size_t> segOff;    // byte offset of each segment
  std::vector<uint64_t> segWords;

  Message(const uint8_t* d, size_t n) : data(d), size(n) {
    if (n < 8) fail("xspn file too short");
    uint32_t nseg;
    std::memcpy(&nseg, d, 4);
    nseg += 1;
    if (nseg == 0 || nseg > 4096) fail("xspn file: implausible segment count");
    size_t hdr = 4 + 4 * (size_t)nseg;
    hdr = (hdr + 7) & ~size_t(7);
    if (hdr > n) fail("xspn file truncated in the segment table");
    size_t off = hdr;
    for (uint32_t i = 0; i < nseg; ++i) {
      uint32_t w;
      std::memcpy(&w, d + 4 + 4 * (size_t)i, 4);
      segOff.push_back(off);
      segWords.push_back(w);
      off += 8 * (size_t)w;
      if (off > n) fail("xspn file truncated: segment exceeds file size");
    }
  }

  uint64_t word(uint32_t seg, uint64_t w) const {
    if (seg >= segWords.size() || w >= segWords[seg]) fail("xspn file: pointer outside its segment");
    uint64_t v;
    std::memcpy(&v, data + segOff[seg] + 8 * w, 8);
    return v;
  }
  const uint8_t* bytes(uint32_t seg, uint64_t w, uint64_t nbytes) const {
    if (seg >= segWords.size() || w > segWords[seg] || nbytes > 8 * (segWords[seg] - w))
      fail("xspn file: object exceeds its segment");
    return data + segOff[seg] + 8 * w;
  }
};

inline int64_t off30(uint64_t p) {
  int64_t v = (int64_t)((p >> 2) & 0x3FFFFFFF);
  return (v & (1 << 29)) ? v - (int64_t(1) << 30) : v;
}

struct Resolved {
  bool null = true;
  uint32_t seg = 0;
  uint64_t ptr = 0;     // the (non-far) pointer word describing the object
  uint64_t target = 0;  // first content word
};

Resolved resolve(const Message& m, uint32_t seg, uint64_t w) {
  Resolved r;
  uint64_t p = m.word(seg, w);
  if (p == 0) return r;
  r.null = false;
  if ((p & 3) != 2) {
    int64_t t = (int64_t)w + 1 + off30(p);
    if (t < 0) fail("xspn file: negative pointer target");
    r.seg = seg; r.ptr = p; r.target = (uint64_t)t;
    return r;
  }
  bool dbl = (p >> 2) & 1;
  uint64_t pad = (p >> 3) & 0x1FFFFFFF;
  uint32_t tseg = (uint32_t)(p >> 32);
  uint64_t q = m.word(tseg, pad);
  if (!dbl) {
    if ((q & 3) == 2) fail("xspn file: far pointer lands on a far pointer");
    int64_t t = (int64_t)pad + 1 + off30(q);
    if (t < 0) fail("xspn file: negative pointer target");
    r.seg = tseg; r.ptr = q; r.target = (uint64_t)t;
    return r;
  }
  uint64_t tag = m.word(tseg, pad + 1);
  if ((q & 3) != 2 || ((q >> 2) & 1)) fail("xspn file: malformed double-far landing pad");
  r.seg = (uint32_t)(q >> 32);
  r.ptr = tag;
  r.target = (q >> 3) & 0x1FFFFFFF;
  return r;
}

struct StructRef {
  const Message* m = nullptr;
  uint32_t seg = 0;
  uint64_t w = 0;
  uint32_t dwords = 0, pwords = 0;
  bool valid() const { return m != nullptr; }

  template <typename T>
  T get(size_t byteOff) const {
    T v{};
    if (!m || byteOff + sizeof(T) > 8 * (size_t)dwords) return v;  // absent field = default 0
    std::memcpy(&v, m->bytes(seg, w, 8 * (uint64_t)dwords) + byteOff, sizeof(T));
    return v;
  }
  Resolved ptr(uint32_t i) const {
    if (!m || i >= pwords) return Resolved{};
    return resolve(*m, seg, w + dwords + i);
  }
  StructRef sub(uint32_t i) const {
    Resolved r = ptr(i);
    StructRef s;
    if (r.null) return s;
    if ((r.ptr & 3) != 0) fail("xspn file: expected a struct pointer");
    s.m = m; s.seg = r.seg; s.w = r.target;
    s.dwords = (uint32_t)((r.ptr >> 32) & 0xFFFF);
    s.pwords = (uint32_t)((r.ptr >> 48) & 0xFFFF);
    m->bytes(s.seg, s.w, 8 * (uint64_t)(s.dwords + s.pwords));
    return s;
  }
  // primitive list: returns pointer + count after checking the element size code
  const uint8_t* list(uint32_t i, unsigned wantCode, unsigned elemBytes, uint64_t* count) const {
    Resolved r = ptr(i);
    *count = 0;
    if (r.null) return nullptr;
    if ((r.ptr & 3) != 1) fail("xspn file: expected a list pointer");
    unsigned code = (unsigned)((r.ptr >> 32) & 7);
    uint64_t cnt = r.ptr >> 35;
    if (cnt == 0) return nullptr;
    if (code != wantCode) fail("xspn file: unexpected list element size");
    *count = cnt;
    return m->bytes(r.seg, r.target, cnt * elemBytes);
  }
  std::string text(uint32_t i) const {
    uint64_t n;
    const uint8_t* p = list(i, 2, 1, &n);
    if (!p || n == 0) return std::string();
    return std::string((const char*)p, (size_t)n - 1);  // drop the NUL terminator
  }
};

struct StructList {
  const Message* m = nullptr;
  uint32_t seg = 0;
  uint64_t first = 0;
  uint64_t count = 0;
  uint32_t dwords = 0, pwords = 0;
  StructRef at(uint64_t k) const {
    StructRef s;
    s.m = m; s.seg = seg; s.w = first + k * (dwords + pwords); s.dwords = dwords; s.pwords = pwords;
    return s;
  }
};

StructList structList(const StructRef& s, uint32_t i) {
  StructList l;
  Resolved r = s.ptr(i);
  if (r.null) return l;
  if ((r.ptr & 3) != 1 || ((r.ptr >> 32) & 7) != 7) fail("xspn file: expected an inline-composite list");
  uint64_t words = r.ptr >> 35;
  uint64_t tag = s.m->word(r.seg, r.target);
  l.m = s.m; l.seg = r.seg; l.first = r.target + 1;
  l.count = (tag >> 2) & 0x3FFFFFFF;
  l.dwords = (uint32_t)((tag >> 32) & 0xFFFF);
  l.pwords = (uint32_t)((tag >> 48) & 0xFFFF);
  if (l.count * (uint64_t)(l.dwords + l.pwords) > words) fail("xspn file: struct list larger than announced");
  s.m->bytes(r.seg, r.target, 8 * (words + 1));
  return l;
}

template <typename T>
void appendList(std::vector<T>& dst, const StructRef& s, uint32_t i, unsigned code) {
  uint64_t n;
  const uint8_t* p = s.list(i, code, sizeof(T), &n);
  size_t old = dst.size();
  dst.resize(old + (size_t)n);
  if (n) std::memcpy(dst.data() + old, p, (size_t)n * sizeof(T));
}

}  // namespace

FeatureType parseFeatureType(const std::string& text) {
  std::smatch match;
  static const std::regex intRegex{R"(([u]?)int([1-9]+))"};
  static const std::regex floatRegex{R"(float([1-9]+))"};
  FeatureType t;
  if (std::regex_match(text, match, intRegex)) {
    t.kind = match[1].length() ? InKind::UInt : InKind::Int;
    t.bits = std::stoi(match[2]);
    if (t.bits != 8 && t.bits != 16 && t.bits != 32 && t.bits != 64)
      fail("Unsupported feature data type " + text);
    return t;
  }
  if (std::regex_match(text, match, floatRegex)) {
    t.kind = InKind::Float;
    t.bits = std::stoi(match[1]);
    if (t.bits != 32 && t.bits != 64) fail("Unsupported floating-point type " + text);
    return t;
  }
  fail("Unsupported feature data type " + text);
}

Model readXspnBytes(const uint8_t* data, size_t size) {
  Message msg(data, size);
  Resolved root = resolve(msg, 0, 0);
  if (root.null || (root.ptr & 3) != 0) fail("xspn file: missing root struct");
  StructRef header;
  header.m = &msg; header.seg = root.seg; header.w = root.target;
  header.dwords = (uint32_t)((root.ptr >> 32) & 0xFFFF);
  header.pwords = (uint32_t)((root.ptr >> 48) & 0xFFFF);
  msg.bytes(header.seg, header.w, 8 * (uint64_t)(header.dwords + header.pwords));

  Model m;
  StructRef model;
  m.isQuery = header.get<uint16_t>(0) == 1;
  if (m.isQuery) {
    StructRef q = header.sub(0);
    if (!q.valid()) fail("xspn file: empty query");
    m.batchSize = q.get<int32_t>(0);
    m.errorKind = q.get<uint16_t>(4);
    m.maxError = q.get<double>(8);
    StructRef joint = q.sub(0);
    if (!joint.valid()) fail("Can only deserialize joint queries");
    m.supportMarginal = joint.get<uint8_t>(0) & 1;
    model = joint.sub(0);
    if (!model.valid()) fail("No model attached to query");
  } else {
    model = header.sub(0);
    if (!model.valid()) fail("xspn file: empty model");
  }
  int32_t rootId = model.get<int32_t>(0);
  m.numFeatures = model.get<int32_t>(4);
  m.name = model.text(0);
  if (m.name.empty()) m.name = "spn_kernel";
  m.featureType = model.text(1);
  m.ftype = parseFeatureType(m.featureType);

  std::vector<int32_t> scope;
  appendList(scope, model, 2, 4);
  std::sort(scope.begin(), scope.end());
  if ((int64_t)scope.size() != m.numFeatures) fail("xspn file: numFeatures does not match the scope");
  std::unordered_map<int32_t, int32_t> colOf;
  for (size_t i = 0; i < scope.size(); ++i) colOf[scope[i]] = (int32_t)i;
  auto column = [&](int32_t fid) {
    auto it = colOf.find(fid);
    if (it == colOf.end()) fail("Leaf node references unknown feature!");
    return it->second;
  };

  StructList nodes = structList(model, 3);
  size_t n = (size_t)nodes.count;
  m.kind.resize(n);
  m.feature.assign(n, -1);
  m.mean.assign(n, 0.0);
  m.stddev.assign(n, 1.0);
  m.childPtr.assign(n + 1, 0);
  m.tabPtr.assign(n + 1, 0);
  m.brkPtr.assign(n + 1, 0);
  std::unordered_map<int32_t, int32_t> indexOf;
  indexOf.reserve(n * 2);
  std::vector<int32_t> ids;
  for (size_t k = 0; k < n; ++k) {
    StructRef nd = nodes.at(k);
    int32_t id = nd.get<int32_t>(0);
    unsigned which = nd.get<uint16_t>(6);
    StructRef body = nd.sub(0);
    if (which > kCategorical) fail("Unsupported node type");
    if (!body.valid() && which != kProduct && which != kSum) fail("xspn file: leaf without a body");
    m.kind[k] = (uint8_t)which;
    size_t e0 = m.childIdx.size();
    if (which == kProduct || which == kSum) {
      ids.clear();
      if (body.valid()) appendList(ids, body, 0, 4);
      for (int32_t c : ids) {
        auto it = indexOf.find(c);
        if (it == indexOf.end()) fail("No definition found for node with ID: " + std::to_string(c));
        m.childIdx.push_back(it->second);
      }
      if (which == kSum) {
        if (body.valid()) appendList(m.weight, body, 1, 5);
        if (m.weight.size() != m.childIdx.size()) fail("Number of weights must match the number of addends!");
      } else {
        m.weight.resize(m.childIdx.size(), 0.0);
      }
    } else if (which == kHistogram) {
      m.feature[k] = column(body.get<int32_t>(4));
      size_t b0 = m.brk.size(), t0 = m.tab.size();
      appendList(m.brk, body, 0, 4);
      appendList(m.tab, body, 1, 5);
      size_t nb = m.brk.size() - b0;
      if (nb < 2) fail("Histogram needs at least one bucket");
      if (m.tab.size() - t0 < nb - 1) fail("Histogram has fewer densities than buckets");
      m.tab.resize(t0 + nb - 1);  // bucket i = [breaks[i], breaks[i+1]) with densities[i]
    } else if (which == kGaussian) {
      m.mean[k] = body.get<double>(0);
      m.stddev[k] = body.get<double>(8);
      m.feature[k] = column(body.get<int32_t>(16));
    } else {
      m.feature[k] = column(body.get<int32_t>(0));
      size_t t0 = m.tab.size();
      appendList(m.tab, body, 0, 5);
      if (m.tab.size() == t0) fail("Categorical leaf without probabilities");
    }
    (void)e0;
    m.childPtr[k + 1] = (int64_t)m.childIdx.size();
    m.tabPtr[k + 1] = (int64_t)m.tab.size();
    m.brkPtr[k + 1] = (int64_t)m.brk.size();
    indexOf[id] = (int32_t)k;  // after the children: a node cannot be its own operand
  }
  auto it = indexOf.find(rootId);
  if (it == indexOf.end()) fail("No definition found for node with ID: " + std::to_string(rootId));
  m.root = it->second;
  return m;
}

Model readXspnFile(const std::string& path) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) fail("Could not open file " + path);
  std::vector<uint8_t> buf;
  std::fseek(f, 0, SEEK_END);
  long sz = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  if (sz < 0) { std::fclose(f); fail("Could not read file " + path); }
  buf.resize((size_t)sz);
  size_t got = sz ? std::fread(buf.data(), 1, (size_t)sz, f) : 0;
  std::fclose(f);
  if (got != (size_t)sz) fail("Could not read file " + path);
  return readXspnBytes(buf.data(), buf.size());
}

void validateModel(const Model& m) {
  if (m.supportMarginal && !m.ftype.isFloat())
    fail("Feature data type must be floating-point to support marginal");
  const size_t n = m.numNodes();
  if (n == 0 || m.root < 0) fail("Model without nodes");
  for (size_t v = 0; v < n; ++v) {
    int64_t lo = m.childPtr[v], hi = m.childPtr[v + 1];
    switch (m.kind[v]) {
      case kProduct:
        if (hi == lo) fail("Number of operands must be at least one");
        break;
      case kSum: {
        if (hi == lo) fail("Number of addends must be greater than zero!");
        double s = 0.0;
        for (int64_t e = lo; e < hi; ++e) s += m.weight[e];
        if (!(std::abs(s - 1.0) <= 1e-6)) fail("Weights must sum up to 1.0 for normalized SPN");
        break;
      }
      case kHistogram: {
        for (int64_t b = m.brkPtr[v]; b + 1 < m.brkPtr[v + 1]; ++b)
          if (m.brk[b + 1] < m.brk[b]) fail("Lower bound must be less or equal to upper bound!");
        break;
      }
      case kCategorical: {
        double s = 0.0;
        for (int64_t t = m.tabPtr[v]; t < m.tabPtr[v + 1]; ++t) s += m.tab[t];
        if (!(std::abs(s - 1.0) <= 1e-6)) fail("Category probabilities should sum to 1.0");
        break;
      }
      default:
        break;
    }
  }
}

}  // namespace spnb
