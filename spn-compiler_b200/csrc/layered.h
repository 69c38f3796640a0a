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

struct LayeredArgs {
  const LayerStepDev* steps;
  const int* features;
  const float4* quad;      // per (feature, k): a, b, c of  a*x^2 + b*x + c  (base-2 log density)
  const float* weights;
  int numSteps;
  int numInputFeatures;    // columns of the input matrix
  int maxDepth;
  int maxLeafFeatures;
  int marginal;
};

size_t layeredSmemBytes(const LayeredArgs& a, int tile);
cudaError_t layeredLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid, int tile,
                          size_t smem, cudaStream_t stream);
cudaError_t layeredOccupancy(int tile, size_t smem, int* blocksPerSM);

}  // namespace spnb
