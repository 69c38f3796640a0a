// Launch interface of the layered (RAT-SPN) kernel, scalar FP32 version (layered.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace spnb {

struct LayerStepDev {
  int op, width, wa, wb;
  int numFeatures, featOffset, constOffset, pad;
  long long paramOffset;   // leaf: first float4 of the region's parameters; inner: first weight
  long long pad2;
};

// Description of one dense region for the tensor-core path: its weights are stored as half-precision
// mma.sync B fragments, [k-step][n-tile][lane] x 4 halves, each sum's row divided by its largest weight
// (the base-2 log of that divisor is added back after the contraction).
struct MmaRegionDev {
  long long fragOffset;   // first uint2 (4 halves) of the region's fragments
  int scaleOffset;        // first float of the per-sum log2 scale
  int numTiles;           // n-tiles of 8 sums
};

struct LayeredArgs {
  const LayerStepDev* steps;
  const int* features;
  const float4* leafParams;   // per (feature, k): (mu, c2, c1, 0) of  c2*(x - mu)^2 + c1  (base-2 log density)
  const float* weights;
  int numSteps;
  int numInputFeatures;    // columns of the input matrix
  int maxDepth;
  int maxLeafFeatures;
  int marginal;
  long long xtLd;          // > 0: `in` is a feature-major float matrix [numInputFeatures][xtLd] made by transposeInputs
  // tensor-core path (null / 0 when absent)
  const MmaRegionDev* mma;     // per step; fragOffset < 0: the step has no fragments (scalar code runs it)
  const uint2* frags;
  const float* scales;
  int split;                   // 1: fragments come in (value, residue) pairs and three MMAs are issued per pair
  int warpgroups;              // factorised tcgen05 kernel: 1, 2 or 4 warpgroups of 128 threads per CTA
  // factorised tcgen05 kernel: the stages (eight features each) of all tensor-core leaf regions in execution
  // order, every region padded to a multiple of four stages: input column (padding: 0) and the offset
  // subtracted from the input.  A leaf region's MmaRegionDev::scaleOffset is its first stage in this list.
  const int* leafCols;
  const float* leafCentres;
  int numLeafStages;
};

size_t layeredSmemBytes(const LayeredArgs& a, int tile);

// Feature-major float copy of a row-major batch: xt[f * ld + s] = (float)in[s * F + f].  The layered kernels
// read one feature of many consecutive samples at a time; from the row-major layout every such read would
// touch a different 32-byte sector per sample.
cudaError_t transposeInputs(int dtypeCode, const void* in, float* xt, size_t n, int numFeatures, size_t ld,
                            cudaStream_t stream);
// The same for float32 rows, plus a feature-major plane of staged codes for the discrete features (see layered.cu).
cudaError_t transposeInputsCoded(const float* in, float* xt, void* codes, int codeBytes, const int4* meta, size_t n,
                                 int numFeatures, size_t ld, cudaStream_t stream);
cudaError_t layeredLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid, int tile,
                          size_t smem, cudaStream_t stream);
cudaError_t layeredOccupancy(int tile, size_t smem, int* blocksPerSM);

// Tensor-core version: CTAs of 256 samples, dense 32 x (32*32) regions contracted with mma.sync (fp16 in,
// fp32 accumulate); everything else as in the scalar kernel.
size_t layeredMmaSmemBytes(const LayeredArgs& a);
cudaError_t layeredMmaLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid,
                             size_t smem, cudaStream_t stream);
cudaError_t layeredMmaOccupancy(size_t smem, int* blocksPerSM);

// tcgen05 / TMEM version (layered_tcf.cu): leaf regions and inner regions both run as tensor-core
// products with (value, residue) half-precision operands.  LayeredArgs::frags holds per leaf region stages of
// four 1 KB k-step blocks (eight features) and per inner region blocks of four 4 KB k-step blocks (128 columns);
// MmaRegionDev::numTiles is the number of stages / blocks.  *status is set to 1 if a bounded wait gave up.
size_t layeredTcfSmemBytes(const LayeredArgs& a);
cudaError_t layeredTcfLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid,
                             size_t smem, int* status, cudaStream_t stream);

// ---- tcgen05 / TMEM kernel with two sample tiles per CTA (layered_tcf_dual.cu) --------------------------------
// Runs layered models whose inner regions are all full width (32 x 32 cross products, at most 32 sums) and
// whose pending left operands fit into shared memory; everything else stays on layeredTcfKernel.
// The region program is the same post-order walk, annotated with where every region's outputs go.
enum DualDest : int {
  kDualDestStack = 0,     // left operand of a later step: a-stack slot `destSlot` in shared memory
  kDualDestOperand = 1,   // right operand of the next step: written as MMA operand rows
  kDualDestRegs = 2,      // left operand of the step after next (its right sibling is one leaf region): registers
  kDualDestRoot = 3       // root part: folded into the running root log-sum
};

struct DualStepDev {
  int op;                 // LayerOp
  int width;              // outputs
  int dest, destSlot;     // DualDest
  int aSrc;               // inner / root part: a-stack slot of the left operand, -1 = registers
  int numBlocks;          // inner: blocks of 128 (k,i) columns; leaf: stages of eight features (0: FP32 loop only)
  long long fragOffset;   // byte offset of the step's weights in LayeredArgs::frags
  int scaleOffset;        // inner: first of 32 per-sum log2 scales
  int stageBase;          // leaf: first stage of the region in DualArgs::leafCols / leafCentres
  int numFeatures, featOffset;   // leaf: FP32 path
  long long paramOffset;  // leaf: first float4 of the region's (mu, c2, c1, 0) parameters
};

struct DualArgs {
  const DualStepDev* steps;
  int numSteps;
  int aSlots;              // a-stack slots per tile in shared memory
  int globalSlots;         // a-stack slots per tile kept in global memory instead (the outermost ones; slot ids below this)
  float* globalStack;      // [grid][2][globalSlots][33][128] floats
  int ringBlocks;          // 16 KB weight blocks in flight (3 or 4)
  int leafRing;            // leaf stages in flight (2 to 4)
  int marginal;
  const unsigned char* frags;   // same blocks as layeredTcfKernel reads
  const float* scales;          // per sum: base-2 log of the largest weight of its row (the one-tile kernel's form)
  const float* scaleMul;        // per sum: that largest weight itself
  const int* leafCols;          // per stage of eight features:
  const float* leafCentres;     //   input column (padding: 0) and the offset subtracted from the input
  int numLeafStages;
  const int* features;          // FP32 leaf path, as in LayeredArgs
  const float4* leafParams;
  long long xtLd;               // leading dimension of the feature-major input copy
  unsigned spinLimit;           // polls after which a barrier wait gives up
  int testWithholdCommit;       // self-test: the issuer leaves out one commit, so that a bounded wait runs out
  int foldScalar;               // 1: the fold uses scalar FMAs instead of packed pairs (fma.rn.f32x2)
};

size_t layeredDualSmemBytes(int aSlots, int ringBlocks, int leafRing);
size_t layeredDualGlobalStackBytes(int grid, int globalSlots);

}  // namespace spnb

#include <string>
#include <vector>

namespace spnb {

struct LayeredPlan;
struct DualProgram {
  std::vector<DualStepDev> steps;
  std::vector<int> cols4;        // DualArgs::leafCols
  std::vector<float> centres4;   // DualArgs::leafCentres
  int aSlots = 0;
};
// Annotates the region program for the two-tile kernel.  Per step of `lp`: fragOffset (in 8-byte units, < 0: the
// step has no tensor-core weights), blocks (128-column blocks of an inner region) and scaleOffset as the
// one-tile kernel uses them; centres per entry of lp.features.  False if the program does not fit the
// kernel (an inner region without tensor weights, or a walk that is not a post-order of binary region trees).
bool buildDualProgram(const LayeredPlan& lp, const std::vector<long long>& fragOffset, const std::vector<int>& blocks,
                      const std::vector<int>& scaleOffset, const std::vector<float>& centres, DualProgram* out);
// {"a_slots":..,"leaf_stages":..,"steps":"..."}: one token per step, for the plan statistics and the tests
std::string dualProgramSummary(const DualProgram& p);
int layeredDualThreads();
cudaError_t layeredDualLaunch(const DualArgs& a, const float* xt, float* out, size_t n, int grid, size_t smem, int* status,
                              cudaStream_t stream);

}  // namespace spnb
