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

}  // namespace spnb
