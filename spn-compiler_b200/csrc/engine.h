// Engine: compile (xspn -> plan file) and execute (plan file -> per-sample log-likelihoods on
// one or several GPUs).  Everything above the C ABI in c_api.cc goes through this class.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "emit.h"
#include "model.h"
#include "plan.h"

namespace spnb {

struct KernelMeta {
  std::string kernelName;
  uint32_t queryType = 1, target = 2, batchSize = 1, numFeatures = 0, bytesPerFeature = 0, numResults = 1,
           bytesPerResult = 4;
  std::string dtype = "float32";
};

// Compile options: the reference's keys (compiler/src/option/GlobalOptions.cpp:14-75) plus the
// engine's own "spnb-*" keys.
struct Options {
  bool logSpace = false;       // "use-log-space" (reference default false; its Python layer passes true)
  bool dumpIR = false;         // "dump-ir": print the generated CUDA source and the plan statistics
  bool collectStats = false;   // "collect-graph-stats"
  std::string statsFile = "/tmp/stats.json";
  int maxTaskSize = -1;        // "maxTaskSize": > 0 caps the DAG nodes per generated function (the reference's task size)
  int optLevel = 3;            // "optLevel"
  std::string kernelMode = "auto";  // "spnb-kernel": auto | unrolled | interp | layered | layered-mma | layered-scalar
  int tile = 0;                // "spnb-tile": threads per CTA (0 = default)
  int minBlocks = 0;           // "spnb-min-blocks": __launch_bounds__ hint of the generated kernel
  int syncEvery = 0;           // "spnb-sync-every"
  int unrollLimit = 300000;    // "spnb-unroll-limit": nodes + edges up to which a DAG is unrolled
  int maxRegisters = 0;        // "spnb-max-registers"
  int gaussForm = 1;           // "spnb-gauss-form"
  int chunkNodes = -1;         // "spnb-chunk-nodes": DAG nodes per generated function (-1 = default, 0 = one function)
  int mmaSplit = 1;            // "spnb-mma-split": 1 = half-precision operands carry their rounding residue (3 MMAs), 0 = plain fp16
  int tcWarpgroups = 1;        // "spnb-tc-warpgroups": warpgroups (128 threads) per CTA of the tensor-memory layered kernel
  int scoped = -1;             // "spnb-scoped": scope-local staging of a chunked generated kernel (-1 automatic, 0 off, 1 on)
  int asyncStage = 1;          // "spnb-async-stage": 0 = never stage the next tile with cp.async while one is evaluated
  int scopeCut = 0;            // "spnb-scope-cut": 1 = end scope-local chunks where the fewest values are alive
  int stageUnroll = 12;         // "spnb-stage-unroll": unroll factor of the scope-local staging loops
  int loadMode = 0;            // "spnb-load-mode": 0 early load, 1 L1 prefetch and load at the first use, 2 early volatile load
  int prefetchSlots = 0;       // "spnb-prefetch-slots": depth of the shared-memory ring operands of earlier chunks are copied into ahead of their use
  int rowStageUnroll = 8;      // "spnb-row-stage-unroll": unroll factor of the row-major staging loop
  int chunkBarrier = 0;        // "spnb-chunk-barrier": 1 = CTA-wide barriers around every chunk's staging with scope-local staging
  int fuseLeaves = 1;          // "spnb-fuse-leaves": fused tables for the discrete leaf children of a product
  int fuseEntries = 32;        // "spnb-fuse-entries": largest fused table, in entries
  int codePlane = 1;           // "spnb-code-plane": 0 = scope-local staging digests discrete inputs itself
  int loadAhead = 0;           // "spnb-load-ahead": nodes between the request of an earlier chunk's value and its first use
  int hoistLoads = 0;          // "spnb-hoist-loads": operands of earlier chunks a scope-local chunk requests at its top
  int scopeBytes = 0;          // "spnb-scope-bytes": staged bytes per sample and chunk (0 = what fits)
  int tcTiles = 2;             // "spnb-tc-tiles": 2 = two sample tiles per CTA where the model allows it, 1 = one tile
  int tcRings = 0;             // "spnb-tc-rings": two digits, weight blocks (2-6) and leaf stages (2-7) in flight in the two-tile kernel; 0 = automatic
  int tcGlobalSlots = -1;      // "spnb-tc-global-slots": pending left operands per tile kept in global instead of shared memory; -1 = automatic
  int tcFoldScalar = 0;        // "spnb-tc-fold": packed (fma.rn.f32x2, default) or scalar FMAs in the two-tile kernel's fold
  long long spinLimit = 0;     // "spnb-spin-limit": polls after which a tensor-core barrier wait gives up (0 = 2^17, about a second)
  int selftestWithhold = 0;    // "spnb-selftest-withhold-commit": 1 = the two-tile kernel leaves out one commit (tests
                               // that a bounded wait runs out and is reported; results of such a plan are invalid)
  int bucketClamp = 0;         // "spnb-bucket-clamp": 1 = histogram buckets by multiply-shift-clamp where exact (no gain measured: off)
  int bucketArith = 0;         // "spnb-bucket-arith": 1 = compute histogram buckets by multiply-shift where exact (measured slower: off)
  int interpSlots = 0;         // "spnb-interp-slots": cap on the interpreter's shared-memory value slots (0 = as many as fit)
  int groupTiles = 0;          // "spnb-group-tiles": tiles per chunk run of a chunked kernel (0 = automatic)
  int tableWindow = 0;         // "spnb-table-window": bytes of shared memory for leaf tables (0 = 64 KB)
  std::vector<std::pair<std::string, std::string>> raw;
};

Options parseOptions(const std::vector<std::pair<std::string, std::string>>& kv);

enum Strategy : int32_t { kUnrolled = 0, kInterpreter = 1, kLayered = 2 };

class Engine {
 public:
  // Compile `queryPath` into `planPath` (empty: a fresh temporary file is chosen and returned).
  static std::string compile(const std::string& queryPath, const Options& opt, const std::string& planPath,
                             KernelMeta* meta);
  static std::unique_ptr<Engine> load(const std::string& planPath);
  ~Engine();

  const KernelMeta& meta() const { return meta_; }
  const std::string& statsJson() const { return statsJson_; }
  const std::string& source() const { return source_; }

  void executeHost(size_t n, const void* in, void* out);
  void executeDevice(int device, size_t n, const void* dIn, void* dOut, cudaStream_t stream);
  void executeDeviceNoAlloc(int device, size_t n, const void* dIn, void* dOut, cudaStream_t stream);
  void executeSharded(const int* devices, int nDevices, size_t n, const void* in, void* out, double* meanOut);
  void setDevice(int device) { hostDevice_ = device; }
  void launchConfig(int device, int* grid, int* block, size_t* smem);
  void deviceStatus(int device);   // synchronises the device; throws if a kernel's bounded wait gave up
  float lastKernelMs() const { return lastKernelMs_; }

 private:
  struct DeviceState;
  Engine() = default;
  DeviceState& state(int device);
  void launch(DeviceState& st, size_t n, const void* dIn, void* dOut, cudaStream_t stream);
  void* scratchFor(DeviceState& st, cudaStream_t stream);
  void checkStatusFlag(DeviceState& st);
  void runHostOnDevice(int device, size_t n, const void* in, void* out, float* kernelMs);

  Model model_;
  Plan plan_;
  KernelMeta meta_;
  Strategy strategy_ = kUnrolled;
  EmitInfo emitInfo_;
  int interpTile_ = 0;
  int interpSlotsCap_ = 0;
  bool layeredScalar_ = false;
  bool mmaSplit_ = true;
  int tcWarpgroups_ = 1;
  int tcTiles_ = 2;
  unsigned spinLimit_ = 1u << 17;   // polls of mbarrier.try_wait, each of which may itself block for microseconds
  int selftestWithhold_ = 0;
  int tcFoldScalar_ = 0;
  int tcRings_ = 0;
  int tcGlobalSlots_ = -1;
  bool bucketClamp_ = false;
  bool layeredTcf_ = false;
  std::string source_;
  std::vector<char> cubin_;
  std::string statsJson_;
  int hostDevice_ = 0;
  float lastKernelMs_ = 0.f;
  std::mutex mu_;
  std::mutex planMu_;
  // allocation-free path (executeDeviceNoAlloc)
  std::mutex noAllocMu_;
  std::unique_ptr<Plan> noAllocPlan_;
  std::vector<int4> noAllocMeta_;
  int noAllocTile_ = 0, noAllocSlots_ = 0, noAllocOptin_ = 0;
  unsigned long long noAllocTag_ = 0;
  std::map<int, std::unique_ptr<DeviceState>> dev_;
};

}  // namespace spnb
