// Issue-rate micro-benchmarks that give the compute denominators of the per-config roofline:
// FP32 fused multiply-adds, SFU transcendentals (ex2.approx / lg2.approx) and FP64 FMAs per second
// on the device the engine runs on.  Each thread keeps eight independent dependency chains so that
// the pipes, not latencies, set the rate.
#include <cuda_runtime.h>

#include "../../include/spnb.h"

namespace {

template <int KIND>
__global__ void __launch_bounds__(256) rateKernel(float* sink, int iters, float seed) {
  float a[8];
  double da[8];
  unsigned long long pa[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    a[j] = seed + (float)(threadIdx.x + j) * 1e-3f;
    da[j] = (double)a[j];
    pa[j] = ((unsigned long long)__float_as_uint(a[j]) << 32) | __float_as_uint(a[j] + 0.25f);
  }
  const unsigned long long pm = ((unsigned long long)__float_as_uint(0.9999f) << 32) | __float_as_uint(0.9999f);
  const unsigned long long pc = ((unsigned long long)__float_as_uint(1e-4f) << 32) | __float_as_uint(1e-4f);
  const float m = 0.9999f, c = 1e-4f;
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (KIND == 0) {
        a[j] = fmaf(a[j], m, c);
      } else if (KIND == 1) {
        float y;
        asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a[j]));
        a[j] = y;
      } else if (KIND == 2) {
        float y;
        asm volatile("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a[j]));
        a[j] = y;
      } else if (KIND == 3) {
        da[j] = fma(da[j], 0.9999, 1e-4);
      } else {
        // packed pair of FP32 FMAs in one instruction (counted as two operations)
        asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pa[j]) : "l"(pa[j]), "l"(pm), "l"(pc));
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += a[j] + (float)da[j] + __uint_as_float((unsigned)pa[j]) + __uint_as_float((unsigned)(pa[j] >> 32));
  if (s == 12345.678f) sink[0] = s;  // never true; keeps the chains alive
}

template <int KIND>
int run(double* opsPerSecond) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SPNB_ERR_CUDA;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return SPNB_ERR_CUDA;
  float* sink = nullptr;
  if (cudaMalloc(&sink, 16) != cudaSuccess) return SPNB_ERR_CUDA;
  const int iters = KIND == 3 ? 4096 : 16384;
  const int grid = sms * 8, block = 256;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  double best = 0.0;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(e0);
    rateKernel<KIND><<<grid, block>>>(sink, iters, 0.5f);
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    double ops = (double)grid * block * 8.0 * iters * (KIND == 4 ? 2.0 : 1.0);
    if (ms > 0.f) best = ops / (ms * 1e-3) > best ? ops / (ms * 1e-3) : best;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(sink);
  cudaError_t e = cudaGetLastError();
  *opsPerSecond = best;
  return (e == cudaSuccess && best > 0.0) ? SPNB_OK : SPNB_ERR_CUDA;
}

}  // namespace

extern "C" int spnb_measure_peak(int kind, double* ops_per_second) {
  if (!ops_per_second) return SPNB_ERR_ARGUMENT;
  switch (kind) {
    case 0: return run<0>(ops_per_second);
    case 1: return run<1>(ops_per_second);
    case 2: return run<2>(ops_per_second);
    case 3: return run<3>(ops_per_second);
    case 4: return run<4>(ops_per_second);
    default: return SPNB_ERR_ARGUMENT;
  }
}
