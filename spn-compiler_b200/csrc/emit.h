// Emits one straight-line CUDA C++ kernel per model from the planned DAG (compiled by NVRTC for
// sm_100a).  This replaces the reference's LoSPN -> GPU dialect -> NVVM -> PTX lowering
// (mlir/lib/Conversion/LoSPNtoGPU/GPUStructurePatterns.cpp:28-152, GPUNodePatterns.cpp:16-509).
#pragma once
#include <string>
#include <vector>

#include "plan.h"

namespace spnb {

struct EmitOptions {
  int tile = 0;            // threads per CTA = samples per tile (0: chosen from the shared-memory budget)
  int minBlocksPerSM = 0;  // __launch_bounds__ hint (0: derived from the tile)
  int syncEvery = 0;       // CTA barrier every this many DAG nodes (0 = never): keeps the warps of a CTA
                           // on the same stretch of the instruction stream
  int gaussForm = 1;       // 1: fma(d, d, c1/c2) * c2 (three instructions); 0: fma(d*d, c2, c1)
  int chunkNodes = 2000;   // DAG nodes per generated function (0: one function)
  bool chunkExact = false; // the caller asked for that size (spnb-chunk-nodes, maxTaskSize): a hard cap; otherwise DAGs
                           // up to one and a half chunk sizes stay in one function and larger ones are cut evenly
  int groupTiles = 0;      // chunked kernels: tiles a chunk runs on back to back (0 or 1: each tile runs all chunks)
  bool useMax3 = true;     // three-input max.f32 (needs a JIT that knows PTX ISA 8.8)
  bool bucketArith = false;  // histogram buckets by multiply-shift where that reproduces the byte table exactly
                             // (off: five ALU instructions per leaf cost more than the shared-memory read they save)
  bool bucketClamp = false;  // ... with the special codes staged so that one clamp replaces the special cases: three
                             // integer instructions instead of a shared-memory read (measured on the 100-feature
                             // histogram model: 8.43 ms either way, so the byte table stays the default)
  int smemTableLimit = 64 * 1024;  // shared-memory window for leaf tables; larger tables are streamed through it
  // Scope-local staging.  When the inputs of 1024 samples do not fit into shared memory at once (hundreds of
  // features), the DAG is cut into chunks whose leaves read few enough features, and every chunk stages only
  // its own features for the tile, from a feature-major float copy of the batch (made by a small kernel before
  // the launch, coalesced to read).  The CTA keeps 1024 threads, so every fetched instruction of the huge
  // straight-line body serves 32 warps.  -1 = automatic (float32 inputs, log space, more than one chunk, and a
  // CTA of 1024 samples impossible otherwise), 0 = never, 1 = whenever the inputs are float32 in log space.
  int scoped = -1;
  int scopeBytes = 0;              // staged bytes per sample and chunk (0 = what fits beside the table window)
  // Where a scope-local chunk ends once its staging budget is used up: 0 = right there; 1 = at the position of its
  // second half where the fewest values are alive (fewer values through scratch, but a third more chunks and
  // with them more re-staged features: measured 89-92 ms against 86.8 ms on the 53 k-node model, so 0 is the default).
  int scopeCut = 0;
  int stageUnroll = 12;             // scope-local staging: global loads a thread keeps in flight
  int loadMode = 0;                // how the early request is made: 0 load, 1 L1 prefetch + load at the use, 2 volatile load
  int prefetchSlots = 0;           // scope-local staging: operands of earlier chunks copied ahead into a shared-memory ring of this many slots (0: loaded at the use)
  int rowStageUnroll = 8;          // row-major staging: global loads a thread keeps in flight
  int chunkBarrier = 0;            // scope-local staging: 1 = CTA-wide barriers around every chunk's staging (all warps in lock step)
  int fuseLeaves = 1;              // discrete leaf children of one product share a table over their combined code (see emit.cc)
  int fuseEntries = 32;            // largest fused table, in entries
  int codePlane = 1;               // scope-local staging: discrete features are staged from a plane of ready-made codes
  int loadAhead = 0;               // chunked kernels request an operand of an earlier chunk this many nodes before its first use
  int hoistLoads = 0;              // scope-local chunks request up to this many operands of earlier chunks at their top
  // Asynchronous double-buffered staging (float32 inputs that are all read as values, log space): tile t + 1 is
  // copied global -> shared with cp.async while tile t is evaluated.  Rows keep their order with an odd stride,
  // so neither the copy nor the body's reads conflict on shared-memory banks and nothing is transposed.
  // Used when two such buffers fit for the CTA size the single-buffer layout would get.  0 = off.
  int asyncStage = 1;
};

struct EmitInfo {
  std::string kernelName;
  int tile = 0;
  int inputStride = 0;      // floats between two features of one sample in shared memory (tile + 1)
  size_t dynamicSmemBytes = 0;
  bool tablesInSmem = false;
  size_t tableEntries = 0;
  int scratchSlots = 0;     // scratch values per CTA thread: cross-chunk values x tiles per group
  bool scoped = false;      // kernel reads a feature-major float copy:  (xt, out, n, tab, lut, scratch, ld)
  int numChunks = 1;
  int codePlaneBytes = 0;   // > 0: the kernel reads staged codes of this width from a plane behind the feature-major copy
  std::vector<double> fusedTable;   // entries that follow the plan's leaf tables in the kernel's table image
  int fusedGroups = 0;
};

std::string emitCuda(const Plan& plan, const EmitOptions& opt, EmitInfo* info);

}  // namespace spnb
