#include "engine.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <set>
#include <sstream>
#include <stdexcept>
#include <thread>

#include "interp.h"
#include "jit.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

[[noreturn]] void fail(const std::string& m) { throw std::runtime_error(m); }

#define CUDA_OK(expr)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (expr);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      fail(std::string("CUDA error: ") + cudaGetErrorString(e_) + " at " #expr);                   \
  } while (0)

// ---- driver API, resolved through the runtime so that the library links without libcuda ---------
struct Driver {
  decltype(&cuModuleLoadData) moduleLoadData = nullptr;
  decltype(&cuModuleUnload) moduleUnload = nullptr;
  decltype(&cuModuleGetFunction) moduleGetFunction = nullptr;
  decltype(&cuFuncSetAttribute) funcSetAttribute = nullptr;
  decltype(&cuLaunchKernel) launchKernel = nullptr;
  decltype(&cuOccupancyMaxActiveBlocksPerMultiprocessor) occupancy = nullptr;
  decltype(&cuGetErrorString) getErrorString = nullptr;

  static Driver& get() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
      auto load = [](const char* name, void** fn) {
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn)
          fail(std::string("cannot resolve CUDA driver entry point ") + name);
      };
      load("cuModuleLoadData", (void**)&d.moduleLoadData);
      load("cuModuleUnload", (void**)&d.moduleUnload);
      load("cuModuleGetFunction", (void**)&d.moduleGetFunction);
      load("cuFuncSetAttribute", (void**)&d.funcSetAttribute);
      load("cuLaunchKernel", (void**)&d.launchKernel);
      load("cuOccupancyMaxActiveBlocksPerMultiprocessor", (void**)&d.occupancy);
      load("cuGetErrorString", (void**)&d.getErrorString);
    });
    return d;
  }
  void check(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return;
    const char* s = nullptr;
    if (getErrorString) getErrorString(r, &s);
    fail(std::string("CUDA driver error: ") + (s ? s : "unknown") + " in " + what);
  }
};

// Makes `device` current for the lifetime of the object and puts the caller's device back afterwards, also
// when an exception unwinds through it.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != device) {
      CUDA_OK(cudaSetDevice(device));
      changed = true;
    }
  }
  ~DeviceGuard() {
    if (changed && prev >= 0) cudaSetDevice(prev);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};

// CUDA events of one host-path call; destroyed on every way out of it.
struct EventSet {
  std::vector<cudaEvent_t> ev;
  cudaEvent_t add(unsigned flags) {
    cudaEvent_t e = nullptr;
    CUDA_OK(cudaEventCreateWithFlags(&e, flags));
    ev.push_back(e);
    return e;
  }
  ~EventSet() {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
};

bool parseBool(const std::string& v) {
  std::string l = v;
  std::transform(l.begin(), l.end(), l.begin(), ::tolower);
  return l == "true" || l == "yes";  // compiler/src/option/Options.cpp:79-82 of the reference
}

int dtypeCode(const FeatureType& t) {
  if (t.kind == InKind::Float) return t.bits == 32 ? DT_F32 : DT_F64;
  bool u = t.kind == InKind::UInt;
  switch (t.bits) {
    case 8: return u ? DT_U8 : DT_I8;
    case 16: return u ? DT_U16 : DT_I16;
    case 32: return u ? DT_U32 : DT_I32;
    default: return u ? DT_U64 : DT_I64;
  }
}

// ---- plan file -----------------------------------------------------------------------------------
const char kMagic[8] = {'S', 'P', 'N', 'B', 'P', 'L', 'N', '6'};

struct Writer {
  std::vector<uint8_t> b;
  void raw(const void* p, size_t n) { b.insert(b.end(), (const uint8_t*)p, (const uint8_t*)p + n); }
  void u64(uint64_t v) { raw(&v, 8); }
  void str(const std::string& s) { u64(s.size()); raw(s.data(), s.size()); }
  void blob(const void* p, size_t n) { u64(n); raw(p, n); }
};
struct Reader {
  const uint8_t* p; size_t n; size_t o = 0;
  void need(size_t k) { if (k > n - o) fail("plan file truncated"); }
  uint64_t u64() { need(8); uint64_t v; std::memcpy(&v, p + o, 8); o += 8; return v; }
  std::string str() { uint64_t k = u64(); need(k); std::string s((const char*)p + o, k); o += k; return s; }
  std::vector<uint8_t> blob() { uint64_t k = u64(); need(k); std::vector<uint8_t> v(p + o, p + o + k); o += k; return v; }
};

std::vector<uint8_t> readFile(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) fail("Could not open file " + path);
  return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

std::string makeStatsJson(const Plan& p, Strategy s, const EmitInfo& ei, int regs, int spill, int interpSlots) {
  std::ostringstream o;
  std::string base = p.stats.toJson();
  base.pop_back();
  o << base << ",\"log_space\":" << (p.logSpace ? "true" : "false") << ",\"strategy\":\""
    << (s == kUnrolled ? "unrolled" : (s == kInterpreter ? "interpreter" : "layered")) << "\",\"tile\":" << ei.tile << ",\"registers\":" << regs
    << ",\"spill_bytes\":" << spill << ",\"smem_bytes\":" << ei.dynamicSmemBytes << ",\"interp_slots\":" << interpSlots
    << ",\"scratch_slots\":" << ei.scratchSlots << ",\"chunks\":" << ei.numChunks << ",\"scoped_staging\":" << (ei.scoped ? "true" : "false") << ",\"table_entries\":" << (p.tabF32.size() + p.tabF64.size()) << ",\"fused_table_entries\":" << ei.fusedTable.size() << ",\"lut_bytes\":" << p.lut.size() << "}";
  return o.str();
}

void parallelCopy(void* dst, const void* src, size_t bytes) {
  // all but two of the host's hardware threads (at most 16), 2 MB or more each: one thread moves about 5 GB/s,
  // the copy engine behind it takes more than 50
  const size_t kMin = 2u << 20;
  const unsigned hw = std::max(6u, std::thread::hardware_concurrency());
  unsigned nt = (unsigned)std::min<size_t>(std::min(16u, hw - 2), bytes / kMin);
  if (nt <= 1) {
    std::memcpy(dst, src, bytes);
    return;
  }
  std::vector<std::thread> th;
  size_t per = (bytes / nt + 63) & ~size_t(63);
  for (unsigned t = 0; t < nt; ++t) {
    size_t lo = (size_t)t * per, hi = std::min(bytes, lo + per);
    if (lo >= hi) break;
    th.emplace_back([=] { std::memcpy((char*)dst + lo, (const char*)src + lo, hi - lo); });
  }
  for (auto& t : th) t.join();
}

}  // namespace

// ---- options --------------------------------------------------------------------------------------
Options parseOptions(const std::vector<std::pair<std::string, std::string>>& kv) {
  static const std::set<std::string> ignored = {
      "gpu-shared-mem", "search-paths", "cpu-vectorize", "vector-library", "use-shuffle", "irOptLevel", "mcOptLevel",
      "slp-max-attempts", "slp-max-successful-iterations", "slp-max-node-size", "slp-max-look-ahead",
      "slp-reorder-dfs", "slp-allow-duplicate-elements", "slp-allow-topological-mixing", "slp-use-xor-chains",
      "delete-temps", "opt-repr", "stopAfter"};
  Options o;
  o.raw = kv;
  bool haveTarget = false;
  for (auto& p : kv) {
    const std::string& k = p.first;
    const std::string& v = p.second;
    if (k == "target") {
      haveTarget = true;
      if (v == "CPU") fail("Target was 'CPU', but this engine only implements the CUDA target");
      if (v != "CUDA") fail("Unknown value '" + v + "' for option target");
    } else if (k == "use-log-space") o.logSpace = parseBool(v);
    else if (k == "dump-ir") o.dumpIR = parseBool(v);
    else if (k == "collect-graph-stats") o.collectStats = parseBool(v);
    else if (k == "graph-stats-file") o.statsFile = v;
    else if (k == "optLevel") o.optLevel = std::atoi(v.c_str());
    else if (k == "maxTaskSize") o.maxTaskSize = std::atoi(v.c_str());
    else if (k == "spnb-kernel") {
      if (v != "auto" && v != "unrolled" && v != "interp" && v != "layered" && v != "layered-scalar" && v != "layered-mma") fail("Unknown value '" + v + "' for option spnb-kernel");
      o.kernelMode = v;
    } else if (k == "spnb-tile") {
      o.tile = std::atoi(v.c_str());
      if (o.tile != 0 && (o.tile < 32 || o.tile > 1024 || o.tile % 32 != 0))
        fail("spnb-tile must be 0 (automatic) or a multiple of 32 between 32 and 1024");
    }
    else if (k == "spnb-min-blocks") o.minBlocks = std::atoi(v.c_str());
    else if (k == "spnb-sync-every") o.syncEvery = std::atoi(v.c_str());
    else if (k == "spnb-unroll-limit") o.unrollLimit = std::atoi(v.c_str());
    else if (k == "spnb-max-registers") o.maxRegisters = std::atoi(v.c_str());
    else if (k == "spnb-gauss-form") o.gaussForm = std::atoi(v.c_str());
    else if (k == "spnb-table-window") o.tableWindow = std::atoi(v.c_str());
    else if (k == "spnb-chunk-nodes") o.chunkNodes = std::atoi(v.c_str());
    else if (k == "spnb-group-tiles") o.groupTiles = std::atoi(v.c_str());
    else if (k == "spnb-interp-slots") o.interpSlots = std::atoi(v.c_str());
    else if (k == "spnb-mma-split") o.mmaSplit = std::atoi(v.c_str());
    else if (k == "spnb-bucket-arith") o.bucketArith = std::atoi(v.c_str());
    else if (k == "spnb-bucket-clamp") o.bucketClamp = std::atoi(v.c_str());
    else if (k == "spnb-tc-warpgroups") {
      o.tcWarpgroups = std::atoi(v.c_str());
      if (o.tcWarpgroups != 1 && o.tcWarpgroups != 2 && o.tcWarpgroups != 4) fail("spnb-tc-warpgroups must be 1, 2 or 4");
    }
    else if (k == "spnb-scoped") o.scoped = std::atoi(v.c_str());
    else if (k == "spnb-async-stage") o.asyncStage = std::atoi(v.c_str());
    else if (k == "spnb-scope-bytes") o.scopeBytes = std::atoi(v.c_str());
    else if (k == "spnb-scope-cut") o.scopeCut = std::atoi(v.c_str());
    else if (k == "spnb-hoist-loads") o.hoistLoads = std::atoi(v.c_str());
    else if (k == "spnb-load-ahead") o.loadAhead = std::atoi(v.c_str());
    else if (k == "spnb-prefetch-slots") {
      o.prefetchSlots = std::atoi(v.c_str());
      if (o.prefetchSlots < 0 || o.prefetchSlots > 32) fail("spnb-prefetch-slots must be between 0 and 32");
    }
    else if (k == "spnb-row-stage-unroll") o.rowStageUnroll = std::atoi(v.c_str());
    else if (k == "spnb-chunk-barrier") o.chunkBarrier = std::atoi(v.c_str());
    else if (k == "spnb-fuse-leaves") o.fuseLeaves = std::atoi(v.c_str());
    else if (k == "spnb-fuse-entries") o.fuseEntries = std::atoi(v.c_str());
    else if (k == "spnb-code-plane") o.codePlane = std::atoi(v.c_str());
    else if (k == "spnb-load-mode") o.loadMode = std::atoi(v.c_str());
    else if (k == "spnb-stage-unroll") o.stageUnroll = std::atoi(v.c_str());
    else if (k == "spnb-tc-tiles") {
      o.tcTiles = std::atoi(v.c_str());
      if (o.tcTiles != 1 && o.tcTiles != 2) fail("spnb-tc-tiles must be 1 or 2");
    } else if (k == "spnb-tc-rings") {
      o.tcRings = std::atoi(v.c_str());
      if (o.tcRings != 0 && (o.tcRings / 10 < 2 || o.tcRings / 10 > 6 || o.tcRings % 10 < 2 || o.tcRings % 10 > 7))
        fail("spnb-tc-rings must be 0 (automatic) or two digits: weight blocks (2-6) and leaf stages (2-7) in flight");
    } else if (k == "spnb-tc-global-slots") {
      o.tcGlobalSlots = std::atoi(v.c_str());
      if (o.tcGlobalSlots < -1 || o.tcGlobalSlots > 8) fail("spnb-tc-global-slots must be -1 (automatic) or 0-8");
    } else if (k == "spnb-tc-fold") {
      if (v != "packed" && v != "scalar") fail("spnb-tc-fold must be packed or scalar");
      o.tcFoldScalar = v == "scalar" ? 1 : 0;
    } else if (k == "spnb-spin-limit") {
      o.spinLimit = std::atoll(v.c_str());
      if (o.spinLimit < 0 || o.spinLimit > (1ll << 30)) fail("spnb-spin-limit must be between 0 and 2^30");
    } else if (k == "spnb-selftest-withhold-commit") o.selftestWithhold = std::atoi(v.c_str());
    else if (!ignored.count(k)) fail("Unknown compile option " + k);
  }
  if (!haveTarget) fail("Missing required option target");
  if (o.tile && (o.tile < 32 || o.tile > 1024 || o.tile % 32)) fail("spnb-tile must be a multiple of 32 in [32, 1024]");
  return o;
}

// ---- compile --------------------------------------------------------------------------------------
std::string Engine::compile(const std::string& queryPath, const Options& opt, const std::string& planPathIn,
                            KernelMeta* metaOut) {
  std::vector<uint8_t> xspn = readFile(queryPath);
  Model m = readXspnBytes(xspn.data(), xspn.size());
  if (!m.isQuery) fail("Cannot compile raw models");  // SPFlowToMLIRDeserializer.cpp:43-45
  validateModel(m);
  Plan plan = buildPlan(m, opt.logSpace);

  Strategy strat;
  const int64_t size = plan.stats.nodes + plan.stats.sumEdges + plan.stats.productEdges;
  LayeredPlan layered;
  if (opt.kernelMode == "layered" || opt.kernelMode == "layered-scalar" || opt.kernelMode == "layered-mma") {
    if (!opt.logSpace || !recogniseLayers(plan.dag, &layered)) fail("spnb-kernel=layered needs a log-space query whose DAG is a layered (RAT-SPN-style) region graph");
    strat = kLayered;
  } else if (opt.kernelMode == "unrolled") strat = kUnrolled;
  else if (opt.kernelMode == "interp") strat = kInterpreter;
  else {
    // very wide sums unroll into code the JIT takes minutes to digest; the interpreter's inner
    // loop handles them well
    int64_t maxFanIn = 0;
    for (size_t v = 0; v < plan.dag.size(); ++v)
      if (plan.dag.kind[v] == kSum) maxFanIn = std::max<int64_t>(maxFanIn, plan.dag.childPtr[v + 1] - plan.dag.childPtr[v]);
    // (linear space: sums up to 256 addends still unroll quickly, they are plain multiply-add chains)
    strat = (size <= opt.unrollLimit && maxFanIn <= (opt.logSpace ? 64 : 256)) ? kUnrolled : kInterpreter;
    // dense layered models too large to unroll get the layered kernel instead of the interpreter
    if (strat == kInterpreter && opt.logSpace && recogniseLayers(plan.dag, &layered)) strat = kLayered;
  }

  EmitInfo ei;
  std::string source;
  JitResult jr;
  if (strat == kUnrolled) {
    EmitOptions eo;
    if (opt.tile) eo.tile = opt.tile;
    if (opt.minBlocks) eo.minBlocksPerSM = opt.minBlocks;
    eo.syncEvery = opt.syncEvery;
    eo.gaussForm = opt.gaussForm;
    // The reference's task partitioner (mlir/lib/Dialect/LoSPN/Passes/LoSPNTaskPartitioner.cpp:36-148) cuts the
    // graph into tasks of at most maxTaskSize operations that hand their results on through [k x N] buffers
    // in global memory.  The equivalent here: functions of at most that many DAG nodes over consecutive
    // stretches of the evaluation order, results crossing a cut through the per-CTA scratch area.
    if (opt.maxTaskSize > 0) { eo.chunkNodes = opt.maxTaskSize; eo.chunkExact = true; }
    if (opt.chunkNodes >= 0) { eo.chunkNodes = opt.chunkNodes; eo.chunkExact = true; }
    eo.groupTiles = opt.groupTiles;
    if (opt.tableWindow) eo.smemTableLimit = std::min(std::max(opt.tableWindow, 1024), 160 * 1024);
    eo.useMax3 = jitVersion() >= 1209;
    eo.bucketArith = opt.bucketArith != 0;
    eo.bucketClamp = opt.bucketClamp != 0;
    eo.scoped = opt.scoped;
    eo.asyncStage = opt.asyncStage;
    eo.scopeBytes = opt.scopeBytes;
    eo.scopeCut = opt.scopeCut;
    eo.hoistLoads = opt.hoistLoads;
    eo.loadAhead = opt.loadAhead;
    eo.codePlane = opt.codePlane;
    eo.fuseLeaves = opt.fuseLeaves;
    eo.fuseEntries = opt.fuseEntries;
    eo.chunkBarrier = opt.chunkBarrier;
    eo.rowStageUnroll = opt.rowStageUnroll;
    eo.prefetchSlots = opt.prefetchSlots;
    eo.loadMode = opt.loadMode;
    eo.stageUnroll = opt.stageUnroll;
    source = emitCuda(plan, eo, &ei);
    if (ei.dynamicSmemBytes > 227 * 1024) fail("Generated kernel needs more shared memory than one SM has; use spnb-kernel=interp or a smaller spnb-tile");
    jr = jitCompile(source, m.name, opt.optLevel, opt.maxRegisters);
  } else {
    ei.tile = opt.tile;  // 0: chosen at load time from the shared-memory budget
  }

  std::string stats = makeStatsJson(plan, strat, ei, jr.registers, jr.spillBytes, plan.numSlots);
  if (opt.dumpIR) {
    std::fprintf(stderr, "// *** spnb plan statistics ***\n%s\n", stats.c_str());
    if (!source.empty()) std::fprintf(stderr, "// *** generated CUDA source ***\n%s\n// *** NVRTC log ***\n%s\n", source.c_str(), jr.log.c_str());
  }
  if (opt.collectStats) {
    // the reference's key set first (what its tooling reads), the engine's own statistics under "spnb"
    std::ofstream f(opt.statsFile);
    std::string ref = plan.stats.toReferenceJson();
    ref.pop_back();
    f << ref << ",\"spnb\":" << stats << "}\n";
  }

  std::string planPath = planPathIn;
  if (planPath.empty()) {
    const char* tmp = std::getenv("TMPDIR");
    std::string templ = std::string(tmp && *tmp ? tmp : "/tmp") + "/spnbXXXXXX.plan";
    std::vector<char> buf(templ.begin(), templ.end());
    buf.push_back(0);
    int fd = mkstemps(buf.data(), 5);
    if (fd < 0) fail("Could not create a temporary plan file");
    close(fd);
    planPath = buf.data();
  }
  Writer w;
  w.raw(kMagic, 8);
  w.u64(opt.raw.size());
  for (auto& kv : opt.raw) { w.str(kv.first); w.str(kv.second); }
  w.u64((uint64_t)strat);
  w.u64((uint64_t)ei.tile);
  w.u64((uint64_t)ei.dynamicSmemBytes);
  w.u64((uint64_t)ei.scratchSlots);
  w.u64((uint64_t)(ei.scoped ? 1 : 0));
  w.u64((uint64_t)ei.numChunks);
  w.u64((uint64_t)ei.codePlaneBytes);
  w.u64((uint64_t)(jr.registers + 1));
  w.u64((uint64_t)(jr.spillBytes + 1));
  w.blob(xspn.data(), xspn.size());
  w.str(source);
  w.blob(jr.cubin.data(), jr.cubin.size());
  w.blob(reinterpret_cast<const uint8_t*>(ei.fusedTable.data()), ei.fusedTable.size() * sizeof(double));
  {
    std::ofstream f(planPath, std::ios::binary | std::ios::trunc);
    if (!f) fail("Could not write plan file " + planPath);
    f.write((const char*)w.b.data(), (std::streamsize)w.b.size());
  }
  if (metaOut) {
    metaOut->kernelName = m.name;
    metaOut->batchSize = (uint32_t)std::max(m.batchSize, 0);
    metaOut->numFeatures = (uint32_t)m.numFeatures;
    metaOut->bytesPerFeature = (uint32_t)m.ftype.bytes();
    metaOut->bytesPerResult = opt.logSpace ? 4 : 8;
    metaOut->dtype = opt.logSpace ? "float32" : "float64";
  }
  return planPath;
}

// ---- per-device state -------------------------------------------------------------------------------
struct Engine::DeviceState {
  int device = 0;
  int smCount = 0;
  CUmodule module = nullptr;
  CUfunction fn = nullptr;
  void* dTab = nullptr;
  void* dLut = nullptr;
  void* dConsts = nullptr;
  int* dProg = nullptr;
  int* dBreaks = nullptr;
  int4* dMeta = nullptr;
  int grid = 0, block = 0;
  size_t smem = 0;
  InterpArgs ia{};
  LayeredArgs la{};
  void* dSteps = nullptr;
  void* dFeat = nullptr;
  void* dQuad = nullptr;
  void* dWeights = nullptr;
  void* dMma = nullptr;
  void* dFrags = nullptr;
  void* dScales = nullptr;
  bool useMma = false;
  bool useTcf = false;
  void* dCentres = nullptr;
  void* dLeafCols = nullptr;
  // two-tile tcgen05 kernel
  bool useDual = false;
  DualArgs da{};
  void* dDualSteps = nullptr;
  void* dDualCols = nullptr;
  void* dDualCentres = nullptr;
  void* dDualScaleMul = nullptr;
  int samplesPerCta = 0;     // samples one CTA takes per step of its tile loop, if not the block size
  size_t layeredChunkRows = 0;   // samples copied feature-major at a time (layered kernels, scoped generated kernels)
  size_t crossBytes = 0;         // scoped generated kernels: bytes of cross-chunk scratch in front of that copy
  int* dStatus = nullptr;
  // per-CTA scratch of a chunked generated kernel, [grid][slots][tile] values; one area per stream,
  // because launches on different streams may overlap on the GPU
  size_t scratchBytes = 0;
  std::map<cudaStream_t, void*> scratch;
  std::mutex scratchMu;
  // host path
  static constexpr int kBuf = 3;
  cudaStream_t streams[kBuf] = {nullptr, nullptr, nullptr};
  void* hIn[kBuf] = {nullptr, nullptr, nullptr};
  void* dIn[kBuf] = {nullptr, nullptr, nullptr};
  size_t stageBytes = 0;
  void* dOut = nullptr;
  void* hOut = nullptr;
  size_t outBytes = 0;
  std::mutex hostMu;  // one host-path call at a time per device: the staging buffers are shared

  ~DeviceState() {
    cudaSetDevice(device);
    for (int i = 0; i < kBuf; ++i) {
      if (streams[i]) cudaStreamDestroy(streams[i]);
      if (hIn[i]) cudaFreeHost(hIn[i]);
      if (dIn[i]) cudaFree(dIn[i]);
    }
    if (dOut) cudaFree(dOut);
    if (hOut) cudaFreeHost(hOut);
    if (dTab) cudaFree(dTab);
    if (dLut) cudaFree(dLut);
    if (dConsts) cudaFree(dConsts);
    if (dProg) cudaFree(dProg);
    if (dBreaks) cudaFree(dBreaks);
    if (dMeta) cudaFree(dMeta);
    for (auto& kv : scratch) cudaFree(kv.second);
    if (dSteps) cudaFree(dSteps);
    if (dFeat) cudaFree(dFeat);
    if (dQuad) cudaFree(dQuad);
    if (dWeights) cudaFree(dWeights);
    if (dMma) cudaFree(dMma);
    if (dFrags) cudaFree(dFrags);
    if (dScales) cudaFree(dScales);
    if (dStatus) cudaFree(dStatus);
    if (dCentres) cudaFree(dCentres);
    if (dLeafCols) cudaFree(dLeafCols);
    if (dDualSteps) cudaFree(dDualSteps);
    if (dDualCols) cudaFree(dDualCols);
    if (dDualCentres) cudaFree(dDualCentres);
    if (dDualScaleMul) cudaFree(dDualScaleMul);
    if (module) Driver::get().moduleUnload(module);
  }
};

Engine::~Engine() = default;

std::unique_ptr<Engine> Engine::load(const std::string& planPath) {
  std::vector<uint8_t> file = readFile(planPath);
  if (file.size() < 8 || std::memcmp(file.data(), kMagic, 8) != 0) fail("Not a spnb plan file: " + planPath);
  Reader r{file.data(), file.size(), 8};
  std::vector<std::pair<std::string, std::string>> kv;
  uint64_t nopt = r.u64();
  for (uint64_t i = 0; i < nopt; ++i) {
    std::string k = r.str();
    std::string v = r.str();
    kv.emplace_back(k, v);
  }
  Options opt = parseOptions(kv);
  std::unique_ptr<Engine> e(new Engine());
  e->strategy_ = (Strategy)r.u64();
  e->emitInfo_.tile = (int)r.u64();
  e->emitInfo_.dynamicSmemBytes = (size_t)r.u64();
  e->emitInfo_.scratchSlots = (int)r.u64();
  e->emitInfo_.scoped = r.u64() != 0;
  e->emitInfo_.numChunks = (int)r.u64();
  e->emitInfo_.codePlaneBytes = (int)r.u64();
  int regs = (int)r.u64() - 1;
  int spill = (int)r.u64() - 1;
  std::vector<uint8_t> xspn = r.blob();
  e->source_ = r.str();
  std::vector<uint8_t> cubin = r.blob();
  e->cubin_.assign(cubin.begin(), cubin.end());
  {
    std::vector<uint8_t> ft = r.blob();
    e->emitInfo_.fusedTable.resize(ft.size() / sizeof(double));
    if (!ft.empty()) std::memcpy(e->emitInfo_.fusedTable.data(), ft.data(), e->emitInfo_.fusedTable.size() * sizeof(double));
  }
  e->model_ = readXspnBytes(xspn.data(), xspn.size());
  e->plan_ = buildPlan(e->model_, opt.logSpace);
  e->emitInfo_.kernelName = "spnb_kernel";
  e->interpTile_ = e->emitInfo_.tile;
  e->interpSlotsCap_ = opt.interpSlots;
  e->layeredScalar_ = opt.kernelMode == "layered-scalar";
  e->mmaSplit_ = opt.mmaSplit != 0;
  e->tcWarpgroups_ = opt.tcWarpgroups;
  e->tcTiles_ = opt.tcTiles;
  if (opt.spinLimit > 0) e->spinLimit_ = (unsigned)opt.spinLimit;
  e->selftestWithhold_ = opt.selftestWithhold;
  e->tcFoldScalar_ = opt.tcFoldScalar;
  e->tcRings_ = opt.tcRings;
  e->tcGlobalSlots_ = opt.tcGlobalSlots;
  e->bucketClamp_ = opt.bucketClamp != 0;
  // layered models run on the tensor-memory kernel unless another layered kernel is asked for by name
  e->layeredTcf_ = opt.kernelMode != "layered-scalar" && opt.kernelMode != "layered-mma";
  e->meta_.kernelName = e->model_.name;
  e->meta_.batchSize = (uint32_t)std::max(e->model_.batchSize, 0);
  e->meta_.numFeatures = (uint32_t)e->model_.numFeatures;
  e->meta_.bytesPerFeature = (uint32_t)e->model_.ftype.bytes();
  e->meta_.bytesPerResult = opt.logSpace ? 4 : 8;
  e->meta_.dtype = opt.logSpace ? "float32" : "float64";
  e->statsJson_ = makeStatsJson(e->plan_, e->strategy_, e->emitInfo_, regs, spill, e->plan_.numSlots);
  if (e->strategy_ == kLayered && e->layeredTcf_) {
    // would the two-tile tensor-core kernel take this model?  (judged from the region widths alone; leaf regions
    // whose parameters leave half-precision range are decided when the plan is set up on a device)
    LayeredPlan lp;
    DualProgram prog;
    bool dual = false;
    if (opt.tcTiles == 2 && opt.tcWarpgroups == 1 && recogniseLayers(e->plan_.dag, &lp)) {
      const size_t ns = lp.steps.size();
      std::vector<long long> frag(ns, 0);
      std::vector<int> blocks(ns, 0), scaleOff(ns, 0);
      for (size_t i = 0; i < ns; ++i) {
        const LayerStep& s = lp.steps[i];
        if (s.op != kLeafRegion) {
          frag[i] = (s.wa == 32 && s.wb == 32 && s.width <= 32) ? 0 : -1;
          blocks[i] = (s.width * 32 + 127) / 128;
        }
      }
      dual = buildDualProgram(lp, frag, blocks, scaleOff, std::vector<float>(lp.features.size(), 0.f), &prog);
    }
    e->statsJson_.pop_back();
    e->statsJson_ += std::string(",\"tc_tiles\":") + (dual ? "2" : "1");
    if (dual) e->statsJson_ += ",\"tc_program\":" + dualProgramSummary(prog);
    e->statsJson_ += "}";
  }
  return e;
}

Engine::DeviceState& Engine::state(int device) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = dev_.find(device);
  if (it != dev_.end()) return *it->second;
  int count = 0;
  cudaError_t ce = cudaGetDeviceCount(&count);
  if (ce != cudaSuccess || count == 0)
    fail("No CUDA device available: the spnb engine has no CPU fallback");
  if (device < 0 || device >= count) fail("CUDA device " + std::to_string(device) + " does not exist");
  DeviceGuard guard(device);
  CUDA_OK(cudaFree(nullptr));
  std::unique_ptr<DeviceState> st(new DeviceState());
  st->device = device;
  cudaDeviceProp prop;
  CUDA_OK(cudaGetDeviceProperties(&prop, device));
  st->smCount = prop.multiProcessorCount;
  const Plan& p = plan_;
  // padded: a streamed table window may be loaded whole even when it starts near the table's end
  auto upload = [&](const void* src, size_t bytes) -> void* {
    void* d = nullptr;
    CUDA_OK(cudaMalloc(&d, bytes + (256u << 10)));
    CUDA_OK(cudaMemset(d, 0, bytes + (256u << 10)));
    if (bytes) CUDA_OK(cudaMemcpy(d, src, bytes, cudaMemcpyHostToDevice));
    return d;
  };
  // the generated kernel's table image: the plan's leaf tables, then the fused tables the emitter added
  const std::vector<double>& fusedTab = emitInfo_.fusedTable;
  if (strategy_ == kUnrolled && !fusedTab.empty()) {
    if (p.logSpace) {
      std::vector<float> img(p.tabF32);
      for (double v : fusedTab) img.push_back((float)v);
      st->dTab = upload(img.data(), img.size() * 4);
    } else {
      std::vector<double> img(p.tabF64);
      img.insert(img.end(), fusedTab.begin(), fusedTab.end());
      st->dTab = upload(img.data(), img.size() * 8);
    }
  } else if (p.logSpace) st->dTab = upload(p.tabF32.data(), p.tabF32.size() * 4);
  else st->dTab = upload(p.tabF64.data(), p.tabF64.size() * 8);
  st->dLut = upload(p.lut.data(), p.lut.size());
  if (strategy_ == kUnrolled) {
    Driver& drv = Driver::get();
    drv.check(drv.moduleLoadData(&st->module, cubin_.data()), "cuModuleLoadData");
    drv.check(drv.moduleGetFunction(&st->fn, st->module, "spnb_kernel"), "cuModuleGetFunction");
    st->block = emitInfo_.tile;
    st->smem = emitInfo_.dynamicSmemBytes;
    if (st->smem > 48 * 1024)
      drv.check(drv.funcSetAttribute(st->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)st->smem),
                "cuFuncSetAttribute");
    int perSM = 0;
    drv.check(drv.occupancy(&perSM, st->fn, st->block, st->smem), "cuOccupancyMaxActiveBlocksPerMultiprocessor");
    if (perSM < 1) fail("Generated kernel does not fit on one SM");
    st->grid = perSM * st->smCount;
    if (emitInfo_.scratchSlots > 0) {
      st->scratchBytes = (size_t)st->grid * emitInfo_.scratchSlots * st->block * (p.logSpace ? 4 : 8);
      st->scratchBytes = (st->scratchBytes + 255) & ~size_t(255);
    }
    if (emitInfo_.scoped) {
      // the feature-major float copy of (a part of) the batch lives behind the cross-chunk values
      st->crossBytes = st->scratchBytes;
      st->layeredChunkRows = 512 * 1024;
      st->scratchBytes += st->layeredChunkRows * (size_t)p.features.size() * 4;
      if (emitInfo_.codePlaneBytes > 0) {
        // ... and behind it the plane of staged codes of the discrete features, made by the same transposition
        st->scratchBytes += st->layeredChunkRows * (size_t)p.numCodeSlots * (size_t)emitInfo_.codePlaneBytes;
        std::vector<int4> meta(p.features.size());
        for (size_t f = 0; f < meta.size(); ++f)
          meta[f] = make_int4(p.features[f].lo, p.features[f].domain, p.features[f].codeSlot,
                              bucketClamp_ && p.features[f].clampCodes ? 1 : 0);
        st->dMeta = (int4*)upload(meta.data(), meta.size() * sizeof(int4));
      }
    }
  } else if (strategy_ == kLayered) {
    LayeredPlan lp;
    if (!recogniseLayers(p.dag, &lp)) fail("plan file says layered, but the model is not");
    std::vector<LayerStepDev> steps(lp.steps.size());
    for (size_t i = 0; i < steps.size(); ++i) {
      const LayerStep& s = lp.steps[i];
      steps[i] = LayerStepDev{s.op, s.width, s.wa, s.wb, s.numFeatures, (int)s.featOffset, 0, 0, (long long)s.paramOffset, 0};
    }
    st->dSteps = upload(steps.data(), steps.size() * sizeof(LayerStepDev));
    st->dFeat = upload(lp.features.data(), lp.features.size() * 4);
    st->dQuad = upload(lp.leafParams.data(), lp.leafParams.size() * 4);
    st->dWeights = upload(lp.weights.data(), lp.weights.size() * 4);
    st->la.steps = (const LayerStepDev*)st->dSteps;
    st->la.features = (const int*)st->dFeat;
    st->la.leafParams = (const float4*)st->dQuad;
    st->la.weights = (const float*)st->dWeights;
    st->la.numSteps = (int)steps.size();
    st->la.numInputFeatures = (int)p.features.size();
    st->la.maxDepth = lp.maxDepth;
    st->la.maxLeafFeatures = lp.maxLeafFeatures;
    st->la.marginal = (p.marginal && p.ftype.isFloat()) ? 1 : 0;
    // Tensor-core path: every full-width region (32 x 32 cross products) gets its weights as half-precision
    // mma.sync B fragments, [k-step][n-tile][lane] x {k, k+1, k+8, k+9}, rows scaled by their largest weight.
    std::vector<MmaRegionDev> mma(steps.size(), MmaRegionDev{-1, 0, 0});
    std::vector<uint2> frags;
    std::vector<float> scales;
    bool anyMma = false;
    std::vector<float> centres(lp.features.size(), 0.f);
    std::vector<int> leafCols;        // flat list of leaf stages (eight slots each), see LayeredArgs::leafCols
    std::vector<float> leafCentres;
    auto halfBits = [](float v, bool residue) -> unsigned {
      __half h = __float2half_rn(v);
      if (residue) h = __float2half_rn(v - __half2float(h));
      unsigned short bits;
      std::memcpy(&bits, &h, 2);
      return bits;
    };
    if (layeredTcf_) {
      // Factorised tensor-memory kernel (layered_tcf.cu).  All blocks are in the K-major core-matrix layout
      // [k-half][row group][row % 8][8 halves]; one row of a k-half is 16 bytes = two uint2.
      for (size_t i = 0; i < steps.size(); ++i) {
        const LayerStep& s = lp.steps[i];
        if (s.width > 32) continue;
        if (s.op == kLeafRegion) {
          // per feature: centre = mean of the components' means; the density c2 (x - mu)^2 + c1 is expanded
          // around it in double:  c2 x'^2 + 2 c2 (centre - mu) x' + c2 (centre - mu)^2 + c1,  x' = x - centre.
          // The expanded terms cancel against each other; with (value, residue) half-precision operands each
          // carries about 22 bits, so a region whose constant term c2 (centre - mu)^2 exceeds 2^12 in magnitude
          // (components many standard deviations apart) would lose more than 2^-10 per leaf and stays on the
          // centred FP32 loop instead.
          const int F = s.numFeatures, K = s.width;
          std::vector<double> ca((size_t)F * K), cb((size_t)F * K), cc((size_t)F * K);
          bool ok = true;
          for (int f = 0; f < F; ++f) {
            double mean = 0.0;
            for (int k = 0; k < K; ++k) mean += (double)lp.leafParams[(s.paramOffset + (size_t)f * K + k) * 4];
            const float m = K ? (float)(mean / K) : 0.f;
            if (!std::isfinite(m)) ok = false;
            centres[(size_t)s.featOffset + f] = m;
            for (int k = 0; k < K; ++k) {
              const float* q = lp.leafParams.data() + (s.paramOffset + (size_t)f * K + k) * 4;
              const double mu = q[0], c2 = q[1], c1 = q[2], dm = (double)m - mu;
              const size_t at = (size_t)f * K + k;
              ca[at] = c2;
              cb[at] = 2.0 * c2 * dm;
              cc[at] = c2 * dm * dm + c1;
              for (double v : {ca[at], cb[at], cc[at]})
                if (!(std::fabs(v) < 60000.0)) ok = false;
              if (!(std::fabs(c2 * dm * dm) <= 4096.0)) ok = false;
            }
          }
          if (!ok) continue;   // the kernel's centred FP32 loop runs the region
          const int nst = (F + 7) / 8;
          mma[i].fragOffset = (long long)frags.size();
          mma[i].scaleOffset = (int)(leafCols.size() / 8);
          mma[i].numTiles = nst;
          for (int st = 0; st < (nst + 3) / 4 * 4; ++st)
            for (int u = 0; u < 8; ++u) {
              const int f = 8 * st + u;
              leafCols.push_back(f < F ? lp.features[(size_t)s.featOffset + f] : 0);
              leafCentres.push_back(f < F ? centres[(size_t)s.featOffset + f] : 0.f);
            }
          for (int st = 0; st < nst; ++st)
            for (int ks = 0; ks < 4; ++ks)
              for (int kh = 0; kh < 2; ++kh)
                for (int k = 0; k < 32; ++k) {
                  const int f = 8 * st + 2 * ks + kh;
                  unsigned h[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                  if (f < F && k < K) {
                    const size_t at = (size_t)f * K + k;
                    const float A = (float)ca[at], B = (float)cb[at], C = (float)cc[at];
                    h[0] = halfBits(A, false); h[1] = h[0]; h[2] = halfBits(A, true);
                    h[3] = halfBits(B, false); h[4] = h[3]; h[5] = halfBits(B, true);
                    h[6] = halfBits(C, false); h[7] = halfBits(C, true);
                  }
                  frags.push_back(uint2{h[0] | (h[1] << 16), h[2] | (h[3] << 16)});
                  frags.push_back(uint2{h[4] | (h[5] << 16), h[6] | (h[7] << 16)});
                }
          anyMma = true;
          continue;
        }
        if (s.wa != 32 || s.wb != 32) continue;
        // inner region: columns (k, i), blocks of 128 columns; per block four k-step chunks:
        // value j 0..15, value j 16..31, residue j 0..15, residue j 16..31
        const int nblk = (s.width * 32 + 127) / 128;
        mma[i].fragOffset = (long long)frags.size();
        mma[i].scaleOffset = (int)scales.size();
        mma[i].numTiles = nblk;
        const float* W = lp.weights.data() + s.paramOffset;
        std::vector<float> inv(32, 0.f);
        for (int k = 0; k < 32; ++k) {
          float mx = 0.f;
          if (k < s.width) for (int q = 0; q < 1024; ++q) mx = std::max(mx, W[(size_t)k * 1024 + q]);
          inv[(size_t)k] = mx > 0.f ? 1.f / mx : 0.f;
          scales.push_back(mx > 0.f ? std::log2(mx) : -INFINITY);
        }
        for (int nb = 0; nb < nblk; ++nb)
          for (int chunk = 0; chunk < 4; ++chunk)
            for (int kh = 0; kh < 2; ++kh)
              for (int r = 0; r < 128; ++r) {
                const int col = 128 * nb + r, k = col >> 5, ii = col & 31;
                const int j0 = 16 * (chunk & 1) + 8 * kh;
                unsigned h[8];
                for (int q = 0; q < 8; ++q) {
                  const float v = k < s.width ? W[(size_t)k * 1024 + ii * 32 + j0 + q] * inv[(size_t)k] : 0.f;
                  h[q] = halfBits(v, chunk >= 2);
                }
                frags.push_back(uint2{h[0] | (h[1] << 16), h[2] | (h[3] << 16)});
                frags.push_back(uint2{h[4] | (h[5] << 16), h[6] | (h[7] << 16)});
              }
        anyMma = true;
      }
    }
    if (!layeredScalar_ && !layeredTcf_) {
      for (size_t i = 0; i < steps.size(); ++i) {
        const LayerStep& s = lp.steps[i];
        if (s.op == kLeafRegion || s.wa != 32 || s.wb != 32 || s.width > 32) continue;
        const int nt = (s.width + 7) / 8;
        mma[i].fragOffset = (long long)frags.size();
        mma[i].scaleOffset = (int)scales.size();
        mma[i].numTiles = nt;
        const float* W = lp.weights.data() + s.paramOffset;
        std::vector<float> inv((size_t)nt * 8, 0.f);
        for (int k = 0; k < nt * 8; ++k) {
          float mx = 0.f;
          if (k < s.width) for (int q = 0; q < 1024; ++q) mx = std::max(mx, W[(size_t)k * 1024 + q]);
          inv[(size_t)k] = mx > 0.f ? 1.f / mx : 0.f;
          scales.push_back(mx > 0.f ? std::log2(mx) : -INFINITY);
        }
        auto h16 = [&](int k, int kk, bool residue) -> unsigned {
          const float v = k < s.width ? W[(size_t)k * 1024 + kk] * inv[(size_t)k] : 0.f;
          __half h = __float2half_rn(v);
          if (residue) h = __float2half_rn(v - __half2float(h));
          unsigned short bits;
          std::memcpy(&bits, &h, 2);
          return bits;
        };
        for (int ks = 0; ks < 64; ++ks)
          for (int t = 0; t < nt; ++t)
            for (int lane = 0; lane < 32; ++lane) {
              const int g = lane >> 2, tig = lane & 3, k = 8 * t + g, kk = 16 * ks + 2 * tig;
              for (int residue = 0; residue < (mmaSplit_ ? 2 : 1); ++residue) {
                uint2 f;
                f.x = h16(k, kk, residue) | (h16(k, kk + 1, residue) << 16);
                f.y = h16(k, kk + 8, residue) | (h16(k, kk + 9, residue) << 16);
                frags.push_back(f);
              }
            }
        anyMma = true;
      }
    }
    if (layeredTcf_) {
      anyMma = true;   // the kernel reads the per-step table for every step
      if (frags.empty()) frags.push_back(uint2{0, 0});
      if (scales.empty()) scales.push_back(0.f);
    }
    if (anyMma) {
      st->dMma = upload(mma.data(), mma.size() * sizeof(MmaRegionDev));
      st->dFrags = upload(frags.data(), frags.size() * sizeof(uint2));
      st->dScales = upload(scales.data(), scales.size() * 4);
      st->la.mma = (const MmaRegionDev*)st->dMma;
      st->la.frags = (const uint2*)st->dFrags;
      st->la.scales = (const float*)st->dScales;
      st->la.split = mmaSplit_ ? 1 : 0;
      st->useMma = true;
      if (layeredTcf_) {
        st->useTcf = true;
        st->la.numLeafStages = (int)(leafCols.size() / 8);
        if (leafCols.empty()) { leafCols.assign(8, 0); leafCentres.assign(8, 0.f); }
        st->dLeafCols = upload(leafCols.data(), leafCols.size() * 4);
        st->dCentres = upload(leafCentres.data(), leafCentres.size() * 4);
        st->la.leafCols = (const int*)st->dLeafCols;
        st->la.leafCentres = (const float*)st->dCentres;
        st->la.warpgroups = tcWarpgroups_;
        CUDA_OK(cudaMalloc(&st->dStatus, sizeof(int)));
        CUDA_OK(cudaMemset(st->dStatus, 0, sizeof(int)));
        // ---- two tiles per CTA, if the program fits that kernel's constraints ----------------------------
        if (tcTiles_ == 2 && tcWarpgroups_ == 1) {
          DualProgram prog;
          std::vector<long long> fragOffsets(steps.size());
          std::vector<int> blockCounts(steps.size()), scaleOffsets(steps.size());
          for (size_t i = 0; i < steps.size(); ++i) {
            fragOffsets[i] = mma[i].fragOffset;
            blockCounts[i] = mma[i].numTiles;
            scaleOffsets[i] = mma[i].scaleOffset;
          }
          if (buildDualProgram(lp, fragOffsets, blockCounts, scaleOffsets, centres, &prog)) {
            std::vector<DualStepDev>& ds = prog.steps;
            std::vector<int>& cols4 = prog.cols4;
            std::vector<float>& centres4 = prog.centres4;
            const size_t ns = ds.size();
            const int maxDepth = prog.aSlots, depth = 0;
            // Ring depths (weight blocks, leaf stages in flight) and where the pending left operands wait.  Measured
            // on the 784-feature model (ms per 2 M samples): 4 + 4 with one pending operand in global memory 201.4,
            // 5 + 4 201.3, 4 + 5 197.0; with all but the innermost pending operand in global memory (33 KB more
            // shared memory for the rings) 4 + 7 187.2, 5 + 6 193.0, 6 + 5 198.0: leaf stages in flight are what pays.
            int ring = 0, leafRing = 0, globalSlots = 0;
            struct Cand { int ring, leafRing, globalSlots; };
            std::vector<Cand> cands;
            if (tcRings_ > 0) {
              const int g = tcGlobalSlots_ >= 0 ? tcGlobalSlots_ : (maxDepth >= 3 ? 1 : 0);
              cands.push_back({tcRings_ / 10, tcRings_ % 10, g});
            } else {
              const int gDeep = std::max(maxDepth - 1, 0), gOne = maxDepth >= 3 ? 1 : 0;
              for (int g : {gDeep, gOne}) {
                if (tcGlobalSlots_ >= 0 && g != gDeep) continue;
                const int gg = tcGlobalSlots_ >= 0 ? tcGlobalSlots_ : g;
                for (int lr : {7, 6, 5, 4, 3, 2}) cands.push_back({4, lr, gg});
                for (int lr : {3, 2}) cands.push_back({3, lr, gg});
              }
            }
            for (const Cand& c : cands) {
              const int g = std::min(c.globalSlots, std::max(maxDepth - 1, 0));
              if (layeredDualSmemBytes(std::max(maxDepth - g, 1), c.ring, c.leafRing) <= (size_t)prop.sharedMemPerBlockOptin) {
                ring = c.ring;
                leafRing = c.leafRing;
                globalSlots = g;
                break;
              }
            }
            const int smemSlots = std::max(maxDepth - globalSlots, 1);
            if (ring && depth == 0) {
              if (cols4.empty()) { cols4.assign(8, 0); centres4.assign(8, 0.f); }
              // per sum the largest weight of its row, the multiplier form of the log2 scales
              std::vector<float> scaleMul(scales.size());
              for (size_t q = 0; q < scales.size(); ++q) scaleMul[q] = std::isfinite(scales[q]) ? std::exp2(scales[q]) : 0.f;
              st->dDualScaleMul = upload(scaleMul.data(), scaleMul.size() * 4);
              st->da.scaleMul = (const float*)st->dDualScaleMul;
              st->da.leafRing = leafRing;
              st->dDualSteps = upload(ds.data(), ds.size() * sizeof(DualStepDev));
              st->dDualCols = upload(cols4.data(), cols4.size() * 4);
              st->dDualCentres = upload(centres4.data(), centres4.size() * 4);
              st->da.steps = (const DualStepDev*)st->dDualSteps;
              st->da.numSteps = (int)ns;
              st->da.aSlots = smemSlots;
              st->da.globalSlots = globalSlots;
              st->da.ringBlocks = ring;
              st->da.marginal = st->la.marginal;
              st->da.frags = (const unsigned char*)st->dFrags;
              st->da.scales = (const float*)st->dScales;
              st->da.leafCols = (const int*)st->dDualCols;
              st->da.leafCentres = (const float*)st->dDualCentres;
              st->da.numLeafStages = (int)(cols4.size() / 8);
              st->da.features = st->la.features;
              st->da.leafParams = st->la.leafParams;
              st->da.spinLimit = spinLimit_;
              st->da.testWithholdCommit = selftestWithhold_;
              st->da.foldScalar = tcFoldScalar_;
              st->useDual = true;
              st->block = layeredDualThreads();
              st->samplesPerCta = 256;
              st->smem = layeredDualSmemBytes(st->da.aSlots, ring, leafRing);
              st->grid = st->smCount;   // one CTA per SM: the kernel owns the SM's tensor memory
              st->layeredChunkRows = 512 * 1024;
              // scratch per stream: the spilled a-stack slots of every CTA, then the feature-major input copy
              st->crossBytes = (layeredDualGlobalStackBytes(st->grid, globalSlots) + 255) & ~size_t(255);
              st->scratchBytes = st->crossBytes + st->layeredChunkRows * (size_t)p.features.size() * 4;
              auto insD = dev_.emplace(device, std::move(st));
              return *insD.first->second;
            }
          }
        }
        st->block = 128;
        st->smem = layeredTcfSmemBytes(st->la);
        if (st->smem > (size_t)prop.sharedMemPerBlockOptin) fail("Layered tcgen05 kernel: region stack too deep for shared memory");
        st->grid = st->smCount;   // one CTA per SM: the kernel owns the SM's tensor memory
        st->layeredChunkRows = 512 * 1024;
        st->scratchBytes = st->layeredChunkRows * (size_t)p.features.size() * 4;
        auto insF = dev_.emplace(device, std::move(st));
        return *insF.first->second;
      }
      st->block = 256;
      st->smem = layeredMmaSmemBytes(st->la);
      if (st->smem > (size_t)prop.sharedMemPerBlockOptin) fail("Layered tensor-core kernel: region stack too deep for shared memory");
      int perSM = 0;
      CUDA_OK(layeredMmaOccupancy(st->smem, &perSM));
      if (perSM < 1) fail("Layered tensor-core kernel does not fit on one SM");
      st->grid = perSM * st->smCount;
    } else {
      int tile = interpTile_ ? interpTile_ : 128;
      while (tile > 32 && layeredSmemBytes(st->la, tile) > (size_t)prop.sharedMemPerBlockOptin) tile /= 2;
      st->block = tile;
      st->smem = layeredSmemBytes(st->la, tile);
      int perSM = 0;
      CUDA_OK(layeredOccupancy(tile, st->smem, &perSM));
      if (perSM < 1) fail("Layered kernel does not fit on one SM");
      st->grid = perSM * st->smCount;
    }
    st->layeredChunkRows = 512 * 1024;
    st->scratchBytes = st->layeredChunkRows * (size_t)p.features.size() * 4;
  } else {
    std::vector<int4> meta(p.features.size());
    for (size_t f = 0; f < meta.size(); ++f)
      meta[f] = make_int4(p.features[f].lo, p.features[f].domain, p.features[f].codeSlot, p.features[f].valueSlot);
    st->dBreaks = (int*)upload(p.groupBreaks.data(), p.groupBreaks.size() * 4);
    st->dMeta = (int4*)upload(meta.data(), meta.size() * sizeof(int4));
    st->ia.tab = st->dTab;
    st->ia.linear = p.logSpace ? 0 : 1;
    const size_t valueBytes = p.logSpace ? 4 : 8;
    st->ia.lut = (const unsigned char*)st->dLut;
    st->ia.breaks = st->dBreaks;
    st->ia.featureMeta = st->dMeta;
    st->ia.numFeatures = (int)p.features.size();
    st->ia.numValueSlots = p.numValueSlots;
    st->ia.numCodeSlots = p.numCodeSlots;
    st->ia.numSlots = p.numSlots;
    st->ia.marginal = p.marginal ? 1 : 0;
    // Tile and shared-memory slot count: the largest tile that leaves room for all slots, or else for
    // at least 48 of them; the remaining slots live in global scratch memory.
    const size_t budget = (size_t)prop.sharedMemPerBlockOptin;
    const int need = p.numSlots;
    int tile = 0, smemSlots = 0;
    for (int t : {256, 128, 64, 32}) {
      if (interpTile_ && t != interpTile_) continue;
      st->ia.numSlots = 0;
      const size_t base = interpSmemBytes(st->ia, t);
      if (base >= budget) continue;
      int fit = (int)std::min<size_t>((budget - base) / ((size_t)t * valueBytes), (size_t)need);
      if (interpSlotsCap_ > 0) fit = std::min(fit, interpSlotsCap_);
      if (fit >= std::min(need, interpSlotsCap_ > 0 ? interpSlotsCap_ : 48)) { tile = t; smemSlots = fit; break; }
    }
    if (!tile) fail("The staged inputs of one warp of samples do not fit into shared memory");
    if (smemSlots < need) {
      std::lock_guard<std::mutex> lock(planMu_);
      if (plan_.numSpillSlots == 0 || plan_.numSmemSlots > smemSlots) buildProgram(plan_, smemSlots);
    }
    st->ia.numSlots = smemSlots;
    st->ia.numSpillSlots = plan_.numSpillSlots;
    st->dProg = (int*)upload(plan_.prog.data(), plan_.prog.size() * 4);
    st->dConsts = upload(plan_.progConsts.data(), plan_.progConsts.size() * 8);
    st->ia.dconst = (const double*)st->dConsts;
    st->ia.prog = st->dProg;
    st->ia.progLen = (int)plan_.prog.size();
    st->block = tile;
    st->smem = interpSmemBytes(st->ia, tile);
    int perSM = 0;
    CUDA_OK(interpOccupancy(dtypeCode(p.ftype), tile, st->smem, &perSM, !p.logSpace));
    if (perSM < 1) fail("Interpreter kernel does not fit on one SM");
    st->grid = perSM * st->smCount;
    st->scratchBytes = (size_t)st->grid * plan_.numSpillSlots * st->block * valueBytes;
  }
  auto ins = dev_.emplace(device, std::move(st));
  return *ins.first->second;
}

void Engine::launchConfig(int device, int* grid, int* block, size_t* smem) {
  DeviceState& st = state(device);
  if (grid) *grid = st.grid;
  if (block) *block = st.block;
  if (smem) *smem = st.smem;
}

// Reads (and clears) the flag the tcgen05 layered kernel raises when one of its bounded waits expires.
// The copy is synchronous, so it also waits for the launches queued before it.
void Engine::checkStatusFlag(DeviceState& st) {
  if (!st.dStatus) return;
  int flag = 0;
  CUDA_OK(cudaMemcpy(&flag, st.dStatus, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag) {
    cudaMemset(st.dStatus, 0, sizeof(int));
    fail("tcgen05 layered kernel: a bounded wait on a tensor-core barrier gave up; results are incomplete");
  }
}

void Engine::deviceStatus(int device) {
  DeviceState& st = state(device);
  DeviceGuard guard(device);
  CUDA_OK(cudaDeviceSynchronize());
  checkStatusFlag(st);
}

// The scratch area used by launches on `stream` (allocated on first use; null if the plan needs none).
void* Engine::scratchFor(DeviceState& st, cudaStream_t stream) {
  if (!st.scratchBytes) return nullptr;
  std::lock_guard<std::mutex> lock(st.scratchMu);
  auto it = st.scratch.find(stream);
  if (it == st.scratch.end()) {
    void* p = nullptr;
    CUDA_OK(cudaMalloc(&p, st.scratchBytes));
    it = st.scratch.emplace(stream, p).first;
  }
  return it->second;
}

void Engine::launch(DeviceState& st, size_t n, const void* dIn, void* dOut, cudaStream_t stream) {
  if (n == 0) return;
  const size_t tiles = (n + (size_t)st.block - 1) / (size_t)st.block;
  const int grid = (int)std::min<size_t>(tiles, (size_t)st.grid);
  if (strategy_ == kUnrolled) {
    void* dScratch = scratchFor(st, stream);
    Driver& drv = Driver::get();
    if (emitInfo_.scoped) {
      // feature-major float copy first (at most layeredChunkRows samples at a time), then the kernel on it
      float* xt = reinterpret_cast<float*>(static_cast<char*>(dScratch) + st.crossBytes);
      const size_t rowBytes = (size_t)meta_.numFeatures * meta_.bytesPerFeature, resBytes = meta_.bytesPerResult;
      for (size_t r0 = 0; r0 < n; r0 += st.layeredChunkRows) {
        const size_t rows = std::min(st.layeredChunkRows, n - r0);
        unsigned long long ld = (rows + 255) / 256 * 256, nn = rows;
        const void* src = (const char*)dIn + r0 * rowBytes;
        void* dst = (char*)dOut + r0 * resBytes;
        if (emitInfo_.codePlaneBytes > 0)
          CUDA_OK(transposeInputsCoded((const float*)src, xt, xt + (size_t)meta_.numFeatures * ld, emitInfo_.codePlaneBytes,
                                       st.dMeta, rows, (int)meta_.numFeatures, ld, stream));
        else
          CUDA_OK(transposeInputs(dtypeCode(plan_.ftype), src, xt, rows, (int)meta_.numFeatures, ld, stream));
        const size_t tilesC = (rows + (size_t)st.block - 1) / (size_t)st.block;
        const int gridC = (int)std::min<size_t>(tilesC, (size_t)st.grid);   // groups of tiles stride over the grid
        void* args[] = {(void*)&xt, (void*)&dst, (void*)&nn, (void*)&st.dTab, (void*)&st.dLut, (void*)&dScratch, (void*)&ld};
        drv.check(drv.launchKernel(st.fn, gridC, 1, 1, st.block, 1, 1, (unsigned)st.smem, (CUstream)stream, args, nullptr),
                  "cuLaunchKernel");
      }
      return;
    }
    unsigned long long nn = n;
    void* args[] = {(void*)&dIn, (void*)&dOut, (void*)&nn, (void*)&st.dTab, (void*)&st.dLut, (void*)&dScratch};
    drv.check(drv.launchKernel(st.fn, grid, 1, 1, st.block, 1, 1, (unsigned)st.smem, (CUstream)stream, args, nullptr),
              "cuLaunchKernel");
  } else if (strategy_ == kLayered) {
    // The batch is first copied into a feature-major float matrix in scratch memory (one area per stream),
    // at most kLayeredChunk samples at a time; the layered kernels then read it coalesced.
    const size_t kLayeredChunk = st.layeredChunkRows;
    char* layeredScratch = (char*)scratchFor(st, stream);
    float* xt = (float*)(layeredScratch + (st.useDual ? st.crossBytes : 0));
    const size_t rowBytes = (size_t)meta_.numFeatures * meta_.bytesPerFeature;
    for (size_t r0 = 0; r0 < n; r0 += kLayeredChunk) {
      const size_t rows = std::min(kLayeredChunk, n - r0);
      const size_t ld = (rows + 255) / 256 * 256;
      const void* src = (const char*)dIn + r0 * rowBytes;
      float* dst = (float*)dOut + r0;
      CUDA_OK(transposeInputs(dtypeCode(plan_.ftype), src, xt, rows, (int)meta_.numFeatures, ld, stream));
      LayeredArgs la = st.la;
      la.xtLd = (long long)ld;
      const size_t perCta = st.samplesPerCta ? (size_t)st.samplesPerCta : (size_t)st.block;
      const size_t tilesC = (rows + perCta - 1) / perCta;
      const int gridC = (int)std::min<size_t>(tilesC, (size_t)st.grid);
      if (st.useDual) {
        DualArgs da = st.da;
        da.xtLd = (long long)ld;
        da.globalStack = (float*)layeredScratch;
        CUDA_OK(layeredDualLaunch(da, xt, dst, rows, gridC, st.smem, st.dStatus, stream));
      } else if (st.useTcf) CUDA_OK(layeredTcfLaunch(la, DT_F32, xt, dst, rows, gridC, st.smem, st.dStatus, stream));
      else if (st.useMma) CUDA_OK(layeredMmaLaunch(la, DT_F32, xt, dst, rows, gridC, st.smem, stream));
      else CUDA_OK(layeredLaunch(la, DT_F32, xt, dst, rows, gridC, st.block, st.smem, stream));
    }
  } else {
    InterpArgs ia = st.ia;
    ia.scratch = scratchFor(st, stream);
    CUDA_OK(interpLaunch(ia, dtypeCode(plan_.ftype), dIn, dOut, n, grid, st.block, st.smem, stream));
  }
}

// Evaluation with no device allocation on the way: the interpreter kernel with model image and spill
// scratch in the library's static device area (interp.cu).  Uses a private copy of the plan whose
// program is built for the tile / slot split chosen here, so the regular path's state is untouched.
void Engine::executeDeviceNoAlloc(int device, size_t n, const void* dIn, void* dOut, cudaStream_t stream) {
  if (!plan_.logSpace) fail("The allocation-free entry point runs the log-space interpreter only");
  if (n == 0) return;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
    fail("No CUDA device available: the spnb engine has no CPU fallback");
  if (device < 0 || device >= count) fail("CUDA device " + std::to_string(device) + " does not exist");
  DeviceGuard guard(device);
  std::lock_guard<std::mutex> lock(noAllocMu_);
  int optin = 0;
  CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  if (!noAllocPlan_ || noAllocOptin_ != optin) {
    std::unique_ptr<Plan> np(new Plan(plan_));
    buildProgram(*np, INT32_MAX);
    InterpArgs ia{};
    ia.numFeatures = (int)np->features.size();
    ia.numValueSlots = np->numValueSlots;
    ia.numCodeSlots = np->numCodeSlots;
    const int need = np->numSlots;
    const int cap = interpSlotsCap_ > 0 ? interpSlotsCap_ : 48;
    int tile = 0, smemSlots = 0;
    for (int t : {256, 128, 64, 32}) {
      if (interpTile_ && t != interpTile_) continue;
      ia.numSlots = 0;
      const size_t base = interpSmemBytes(ia, t);
      if (base >= (size_t)optin) continue;
      int fit = (int)std::min<size_t>(((size_t)optin - base) / ((size_t)t * 4), (size_t)need);
      if (interpSlotsCap_ > 0) fit = std::min(fit, interpSlotsCap_);
      if (fit >= std::min(need, cap)) { tile = t; smemSlots = fit; break; }
    }
    if (!tile) fail("The staged inputs of one warp of samples do not fit into shared memory");
    if (smemSlots < need) buildProgram(*np, smemSlots);
    noAllocMeta_.resize(np->features.size());
    for (size_t f = 0; f < noAllocMeta_.size(); ++f)
      noAllocMeta_[f] = make_int4(np->features[f].lo, np->features[f].domain, np->features[f].codeSlot, np->features[f].valueSlot);
    noAllocPlan_ = std::move(np);
    static std::atomic<unsigned long long> nextTag{1};
    noAllocTag_ = nextTag.fetch_add(1);
    noAllocTile_ = tile;
    noAllocSlots_ = smemSlots;
    noAllocOptin_ = optin;
  }
  const Plan& p = *noAllocPlan_;
  InterpArgs ia{};
  ia.progLen = (int)p.prog.size();
  ia.numFeatures = (int)p.features.size();
  ia.numValueSlots = p.numValueSlots;
  ia.numCodeSlots = p.numCodeSlots;
  ia.numSlots = noAllocSlots_;
  ia.numSpillSlots = p.numSpillSlots;
  ia.marginal = p.marginal ? 1 : 0;
  InterpImage img;
  img.prog = p.prog.data();         img.progBytes = p.prog.size() * 4;
  img.tab = p.tabF32.data();        img.tabBytes = p.tabF32.size() * 4;
  img.lut = p.lut.data();           img.lutBytes = p.lut.size();
  img.breaks = p.groupBreaks.data(); img.breaksBytes = p.groupBreaks.size() * 4;
  img.meta = noAllocMeta_.data();   img.metaBytes = noAllocMeta_.size() * sizeof(int4);
  img.tag = noAllocTag_;
  const char* why = nullptr;
  cudaError_t e = interpLaunchStatic(img, ia, dtypeCode(plan_.ftype), dIn, (float*)dOut, n, noAllocTile_, device, stream, &why);
  if (e != cudaSuccess) fail(why ? std::string("spnb_execute_device_noalloc: ") + why : std::string("CUDA error: ") + cudaGetErrorString(e));
}

void Engine::executeDevice(int device, size_t n, const void* dIn, void* dOut, cudaStream_t stream) {
  DeviceState& st = state(device);
  DeviceGuard guard(device);
  launch(st, n, dIn, dOut, stream);
}

// Host-resident batch on one device: chunks are copied to pinned staging (unless the caller's
// buffer is already pinned), sent with cudaMemcpyAsync and evaluated on rotating streams so that
// copy-in, kernel and copy-out of neighbouring chunks overlap.
void Engine::runHostOnDevice(int device, size_t n, const void* in, void* out, float* kernelMs) {
  if (kernelMs) *kernelMs = 0.f;
  if (n == 0) return;
  DeviceState& st = state(device);
  std::lock_guard<std::mutex> hostLock(st.hostMu);
  DeviceGuard guard(device);
  const size_t rowBytes = (size_t)meta_.numFeatures * meta_.bytesPerFeature;
  const size_t resBytes = meta_.bytesPerResult;
  size_t chunkRows = std::max<size_t>((size_t)(48u << 20) / std::max<size_t>(rowBytes, 1), 4096);
  chunkRows = (chunkRows / (size_t)st.block + 1) * (size_t)st.block;
  chunkRows = std::min(chunkRows, n);
  const size_t nChunks = (n + chunkRows - 1) / chunkRows;

  cudaPointerAttributes ai{}, ao{};
  bool inPinned = cudaPointerGetAttributes(&ai, in) == cudaSuccess && ai.type == cudaMemoryTypeHost;
  bool outPinned = cudaPointerGetAttributes(&ao, out) == cudaSuccess && ao.type == cudaMemoryTypeHost;
  cudaGetLastError();

  const int nbuf = (int)std::min<size_t>(DeviceState::kBuf, nChunks);
  const size_t needStage = chunkRows * rowBytes;
  if (needStage > st.stageBytes) {
    for (int b = 0; b < DeviceState::kBuf; ++b) {
      if (st.hIn[b]) { cudaFreeHost(st.hIn[b]); st.hIn[b] = nullptr; }
      if (st.dIn[b]) { cudaFree(st.dIn[b]); st.dIn[b] = nullptr; }
    }
    st.stageBytes = 0;
  }
  for (int b = 0; b < nbuf; ++b) {
    if (!st.streams[b]) CUDA_OK(cudaStreamCreateWithFlags(&st.streams[b], cudaStreamNonBlocking));
    if (!st.dIn[b]) CUDA_OK(cudaMalloc(&st.dIn[b], needStage));
    if (!inPinned && !st.hIn[b]) CUDA_OK(cudaHostAlloc(&st.hIn[b], needStage, cudaHostAllocDefault));
  }
  st.stageBytes = std::max(st.stageBytes, needStage);
  if (n * resBytes > st.outBytes) {
    if (st.dOut) cudaFree(st.dOut);
    if (st.hOut) cudaFreeHost(st.hOut);
    st.dOut = st.hOut = nullptr;
    CUDA_OK(cudaMalloc(&st.dOut, n * resBytes));
    st.outBytes = n * resBytes;
  }
  if (!outPinned && !st.hOut) CUDA_OK(cudaHostAlloc(&st.hOut, st.outBytes, cudaHostAllocDefault));

  EventSet events;
  std::vector<cudaEvent_t> k0(nChunks), k1(nChunks), done(nChunks);
  for (size_t c = 0; c < nChunks; ++c) {
    k0[c] = events.add(cudaEventDefault);
    k1[c] = events.add(cudaEventDefault);
    done[c] = events.add(cudaEventDisableTiming);
  }
  char* hostOut = outPinned ? (char*)out : (char*)st.hOut;
  size_t drained = 0;  // chunks whose results have been handed to the caller
  auto drain = [&](size_t upto) {
    for (; drained < upto; ++drained) {
      CUDA_OK(cudaEventSynchronize(done[drained]));
      if (!outPinned) {
        size_t r0 = drained * chunkRows, rows = std::min(chunkRows, n - r0);
        std::memcpy((char*)out + r0 * resBytes, hostOut + r0 * resBytes, rows * resBytes);
      }
    }
  };
  for (size_t c = 0; c < nChunks; ++c) {
    const int b = (int)(c % (size_t)nbuf);
    const size_t r0 = c * chunkRows, rows = std::min(chunkRows, n - r0);
    if (c >= (size_t)nbuf) drain(c - nbuf + 1);  // buffer b is free once its previous chunk is done
    const char* src = (const char*)in + r0 * rowBytes;
    if (!inPinned) {
      parallelCopy(st.hIn[b], src, rows * rowBytes);
      src = (const char*)st.hIn[b];
    }
    cudaStream_t s = st.streams[b];
    CUDA_OK(cudaMemcpyAsync(st.dIn[b], src, rows * rowBytes, cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaEventRecord(k0[c], s));
    launch(st, rows, st.dIn[b], (char*)st.dOut + r0 * resBytes, s);
    CUDA_OK(cudaEventRecord(k1[c], s));
    CUDA_OK(cudaMemcpyAsync(hostOut + r0 * resBytes, (char*)st.dOut + r0 * resBytes, rows * resBytes,
                            cudaMemcpyDeviceToHost, s));
    CUDA_OK(cudaEventRecord(done[c], s));
  }
  drain(nChunks);
  checkStatusFlag(st);
  float total = 0.f;
  for (size_t c = 0; c < nChunks; ++c) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, k0[c], k1[c]) == cudaSuccess) total += ms;
  }
  if (kernelMs) *kernelMs = total;
}

void Engine::executeHost(size_t n, const void* in, void* out) {
  float ms = 0.f;
  runHostOnDevice(hostDevice_, n, in, out, &ms);
  lastKernelMs_ = ms;
}

void Engine::executeSharded(const int* devices, int nDevices, size_t n, const void* in, void* out, double* meanOut) {
  if (nDevices <= 0) fail("executeSharded needs at least one device");
  const size_t rowBytes = (size_t)meta_.numFeatures * meta_.bytesPerFeature;
  const size_t resBytes = meta_.bytesPerResult;
  // contiguous row blocks, sizes rounded to 1024 samples so that every shard starts tile-aligned
  size_t per = (n + (size_t)nDevices - 1) / (size_t)nDevices;
  per = (per + 1023) / 1024 * 1024;
  for (int i = 0; i < nDevices; ++i) state(devices[i]);  // create states up front, serially
  std::vector<std::thread> th;
  std::vector<std::string> errors((size_t)nDevices);
  std::vector<float> ms((size_t)nDevices, 0.f);
  for (int i = 0; i < nDevices; ++i) {
    size_t r0 = std::min(n, (size_t)i * per), r1 = std::min(n, r0 + per);
    if (r0 >= r1) continue;
    th.emplace_back([&, i, r0, r1] {
      try {
        runHostOnDevice(devices[i], r1 - r0, (const char*)in + r0 * rowBytes, (char*)out + r0 * resBytes, &ms[(size_t)i]);
      } catch (const std::exception& e) {
        errors[(size_t)i] = e.what();
      }
    });
  }
  for (auto& t : th) t.join();
  for (auto& e : errors)
    if (!e.empty()) fail(e);
  lastKernelMs_ = *std::max_element(ms.begin(), ms.end());
  if (meanOut) {
    double s = 0.0;
    if (resBytes == 4) for (size_t i = 0; i < n; ++i) s += ((const float*)out)[i];
    else for (size_t i = 0; i < n; ++i) s += ((const double*)out)[i];
    *meanOut = n ? s / (double)n : 0.0;
  }
}

}  // namespace spnb
