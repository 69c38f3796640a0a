// Layered (RAT-SPN-style) SPN evaluation, scalar FP32 version: the checking path for the dense sum
// layers and, until the tensor-core version exists, the path that runs them.
//
// One thread per sample, CTAs of `tile` samples.  The region tree is walked in post-order as a stack
// machine whose entries are the (up to 32) outputs of one region, kept in shared memory [level][k][tile]:
//   leaf region   out_k = sum_f c2_kf (x_f - mu_kf)^2 + c1_kf        (factorised Gaussians, base-2 logs)
//   inner region  out_k = ma + mb + log2( sum_i ea_i * sum_j W_k[i,j] * eb_j ),  ea = 2^(a - ma), eb = 2^(b - mb)
// i.e. the cross products of two child regions are never materialised: 2^(a_i + b_j - ma - mb) factorises
// into ea_i * eb_j, which turns wa*wb exponentials per sum into wa + wb per region and leaves a small
// dense contraction per sum.  Weights are streamed through shared memory one sum at a time and are read
// by all threads with broadcast 128-bit loads.
// In the reference these are ordinary sum / product nodes lowered one by one
// (mlir/lib/Conversion/LoSPNtoGPU/GPUNodePatterns.cpp:164-226); the arithmetic here is the same sums in a
// different association order.
#include <cuda_runtime.h>
#include <stdint.h>

#include "interp.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

constexpr int KMAX = 32;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2f(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// shared memory: [stack float x maxDepth*KMAX*tile][wbuf float x KMAX*KMAX][pbuf float4 x maxLeafFeatures*KMAX]
template <typename in_t, bool MARGINAL>
__global__ void __launch_bounds__(256) layeredKernel(LayeredArgs a, const in_t* __restrict__ in, float* __restrict__ out,
                                                      unsigned long long n) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned T = blockDim.x;
  float* stack = reinterpret_cast<float*>(smem_raw);
  float* wbuf = stack + (size_t)a.maxDepth * KMAX * T;
  float4* pbuf = reinterpret_cast<float4*>(wbuf + KMAX * KMAX);
  const unsigned F = a.numInputFeatures;

  const unsigned long long ntiles = (n + T - 1) / T;
  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const unsigned long long row = tile * T + tid;
    const bool live = row < n;
    const in_t* __restrict__ x = in + (a.xtLd ? 0 : (live ? row : 0) * F);
    // feature-major float copy of the batch (see transposeInputs): consecutive samples are consecutive floats
    const float* __restrict__ xT = reinterpret_cast<const float*>(in) + (live ? row : 0);
    int sp = 0;
    float rootM = __int_as_float(0xff800000), rootS = 0.f;
    for (int si = 0; si < a.numSteps; ++si) {
      const LayerStepDev s = a.steps[si];
      if (s.op == kLeafRegion) {
        const int cnt = s.numFeatures * s.width;
        __syncthreads();
        for (int i = tid; i < cnt; i += T) pbuf[i] = a.leafParams[s.paramOffset + i];
        __syncthreads();
        float acc[KMAX];
#pragma unroll
        for (int k = 0; k < KMAX; ++k) acc[k] = 0.f;
        // inputs are fetched eight features ahead: the loads of one batch are independent, so their latency
        // overlaps instead of sitting in front of every feature's 32 updates
        for (int f0 = 0; f0 < s.numFeatures; f0 += 8) {
          float xpre[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int fu = f0 + u < s.numFeatures ? f0 + u : s.numFeatures - 1;
            const int col = __ldg(a.features + s.featOffset + fu);
            xpre[u] = a.xtLd ? xT[(size_t)col * a.xtLd] : (float)x[col];
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int f = f0 + u;
            if (f < s.numFeatures) {
              float xv = xpre[u];
              float m = 1.f;
              if (MARGINAL && xv != xv) { xv = 0.f; m = 0.f; }
              const float4* p = pbuf + f * s.width;
              if (s.width == KMAX) {   // full-width region: no guards, the 32 chains interleave freely
    #pragma unroll
                for (int k = 0; k < KMAX; ++k) {
                  const float4 q = p[k];
                  const float dx = xv - q.x;
                  const float t = fmaf(dx * dx, q.y, q.z);
                  acc[k] = MARGINAL ? fmaf(m, t, acc[k]) : acc[k] + t;
                }
              } else {
    #pragma unroll
                for (int k = 0; k < KMAX; ++k) {
                  if (k < s.width) {
                    const float4 q = p[k];
                    const float dx = xv - q.x;
                  const float t = fmaf(dx * dx, q.y, q.z);
                    acc[k] = MARGINAL ? fmaf(m, t, acc[k]) : acc[k] + t;
                  }
                }
              }
            }
          }
        }
        float* dst = stack + (size_t)sp * KMAX * T + tid;
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
          if (k < s.width) dst[k * T] = acc[k];
        ++sp;
      } else {
        const float* pa = stack + (size_t)(sp - 2) * KMAX * T + tid;
        const float* pb = stack + (size_t)(sp - 1) * KMAX * T + tid;
        float ea[KMAX], eb[KMAX];
        float ma = __int_as_float(0xff800000), mb = ma;
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          ea[i] = i < s.wa ? pa[i * T] : __int_as_float(0xff800000);
          eb[i] = i < s.wb ? pb[i * T] : __int_as_float(0xff800000);
          ma = fmaxf(ma, ea[i]);
          mb = fmaxf(mb, eb[i]);
        }
        const float sa = ma == __int_as_float(0xff800000) ? 0.f : ma;
        const float sb = mb == __int_as_float(0xff800000) ? 0.f : mb;
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          ea[i] = ex2f(ea[i] - sa);
          eb[i] = ex2f(eb[i] - sb);
        }
        const int per = s.wa * s.wb;
        float* dst = stack + (size_t)(sp - 2) * KMAX * T + tid;   // the operands are in registers now
        for (int k = 0; k < s.width; ++k) {
          __syncthreads();
          const float* w = a.weights + s.paramOffset + (long long)k * per;
          for (int i = tid; i < per; i += T) wbuf[i] = __ldg(w + i);
          __syncthreads();
          float acc = 0.f;
          if (s.wa == KMAX && s.wb == KMAX) {
            // full 32 x 32 block: four independent partial sums per row, rows unrolled without guards
            float acc2 = 0.f;
#pragma unroll
            for (int i = 0; i < KMAX; ++i) {
              const float4* wr = reinterpret_cast<const float4*>(wbuf + i * KMAX);
              float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
#pragma unroll
              for (int j = 0; j < KMAX / 4; ++j) {
                const float4 q = wr[j];
                t0 = fmaf(q.x, eb[4 * j], t0);
                t1 = fmaf(q.y, eb[4 * j + 1], t1);
                t2 = fmaf(q.z, eb[4 * j + 2], t2);
                t3 = fmaf(q.w, eb[4 * j + 3], t3);
              }
              if (i & 1) acc2 = fmaf(ea[i], (t0 + t1) + (t2 + t3), acc2);
              else acc = fmaf(ea[i], (t0 + t1) + (t2 + t3), acc);
            }
            acc += acc2;
          } else if ((s.wb & 3) == 0) {
#pragma unroll
            for (int i = 0; i < KMAX; ++i) {
              if (i < s.wa) {
                const float4* wr = reinterpret_cast<const float4*>(wbuf + i * s.wb);
                float t = 0.f;
#pragma unroll
                for (int j = 0; j < KMAX / 4; ++j) {
                  if (4 * j < s.wb) {
                    const float4 q = wr[j];
                    t = fmaf(q.x, eb[4 * j], t);
                    t = fmaf(q.y, eb[4 * j + 1], t);
                    t = fmaf(q.z, eb[4 * j + 2], t);
                    t = fmaf(q.w, eb[4 * j + 3], t);
                  }
                }
                acc = fmaf(ea[i], t, acc);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < KMAX; ++i) {
              if (i < s.wa) {
                float t = 0.f;
#pragma unroll
                for (int j = 0; j < KMAX; ++j)
                  if (j < s.wb) t = fmaf(wbuf[i * s.wb + j], eb[j], t);
                acc = fmaf(ea[i], t, acc);
              }
            }
          }
          const float r = ma + mb + lg2f(acc);
          if (s.op == kInnerRegion) {
            dst[k * T] = r;
          } else {  // root part: fold into the running log-sum
            if (r > rootM) {
              rootS = rootS * ex2f(rootM - r) + 1.f;
              rootM = r;
            } else if (r == r && r != __int_as_float(0xff800000)) {
              rootS += ex2f(r - rootM);
            } else if (r != r) {
              rootS = r;
            }
          }
        }
        sp -= (s.op == kInnerRegion) ? 1 : 2;
      }
    }
    if (live) out[row] = (rootM + lg2f(rootS)) * 0x1.62e43p-1f;
  }
}

template <typename in_t>
cudaError_t launchT(const LayeredArgs& a, const void* in, float* out, size_t n, int grid, int tile, size_t smem,
                    cudaStream_t stream) {
  auto run = [&](auto kernel) -> cudaError_t {
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(kernel), smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, tile, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n);
    return cudaGetLastError();
  };
  return a.marginal ? run(layeredKernel<in_t, true>) : run(layeredKernel<in_t, false>);
}

}  // namespace

namespace {
template <typename in_t>
__global__ void transposeKernel(const in_t* __restrict__ in, float* __restrict__ xt, unsigned long long n, int F,
                                unsigned long long ld) {
  __shared__ float tileBuf[32][33];
  const unsigned long long s0 = (unsigned long long)blockIdx.x * 32;
  const int f0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const unsigned long long srow = s0 + r;
    const int f = f0 + threadIdx.x;
    tileBuf[r][threadIdx.x] = (srow < n && f < F) ? (float)in[srow * F + f] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int f = f0 + r;
    const unsigned long long srow = s0 + threadIdx.x;
    if (f < F && srow < ld) xt[(unsigned long long)f * ld + srow] = tileBuf[threadIdx.x][r];
  }
}
// float32 rows -> feature-major floats plus, for the discrete features, a feature-major plane of staged codes
// (0 missing, 1 outside the domain, 2 + (x - lo) otherwise; with clamped special codes: 65535 / domain + 2):
// codes[slot * ld + s], slot = meta[f].z (-1: no codes for this feature), meta[f] = (lo, domain, slot, clamped)
template <typename code_t>
__global__ void transposeCodedKernel(const float* __restrict__ in, float* __restrict__ xt, code_t* __restrict__ codes,
                                     const int4* __restrict__ meta, unsigned long long n, int F, unsigned long long ld) {
  __shared__ float tileBuf[32][33];
  const unsigned long long s0 = (unsigned long long)blockIdx.x * 32;
  const int f0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const unsigned long long srow = s0 + r;
    const int f = f0 + threadIdx.x;
    tileBuf[r][threadIdx.x] = (srow < n && f < F) ? in[srow * F + f] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int f = f0 + r;
    const unsigned long long srow = s0 + threadIdx.x;
    if (f < F && srow < ld) {
      const float v = tileBuf[threadIdx.x][r];
      xt[(unsigned long long)f * ld + srow] = v;
      const int4 m = meta[f];
      if (m.z >= 0) {
        const unsigned rr = (unsigned)__float2int_rz(v) - (unsigned)m.x;
        int code = rr < (unsigned)m.y ? (int)rr + 2 : (m.w ? m.y + 2 : 1);
        if (v != v) code = m.w ? 65535 : 0;
        codes[(unsigned long long)m.z * ld + srow] = (code_t)code;
      }
    }
  }
}
template <typename in_t>
cudaError_t transposeT(const void* in, float* xt, size_t n, int F, size_t ld, cudaStream_t stream) {
  dim3 grid((unsigned)((ld + 31) / 32), (unsigned)((F + 31) / 32)), block(32, 8);
  transposeKernel<in_t><<<grid, block, 0, stream>>>(static_cast<const in_t*>(in), xt, n, F, ld);
  return cudaGetLastError();
}
}  // namespace

cudaError_t transposeInputs(int dtypeCode, const void* in, float* xt, size_t n, int F, size_t ld, cudaStream_t stream) {
  switch (dtypeCode) {
    case DT_U8: return transposeT<uint8_t>(in, xt, n, F, ld, stream);
    case DT_I8: return transposeT<int8_t>(in, xt, n, F, ld, stream);
    case DT_U16: return transposeT<uint16_t>(in, xt, n, F, ld, stream);
    case DT_I16: return transposeT<int16_t>(in, xt, n, F, ld, stream);
    case DT_U32: return transposeT<uint32_t>(in, xt, n, F, ld, stream);
    case DT_I32: return transposeT<int32_t>(in, xt, n, F, ld, stream);
    case DT_U64: return transposeT<uint64_t>(in, xt, n, F, ld, stream);
    case DT_I64: return transposeT<int64_t>(in, xt, n, F, ld, stream);
    case DT_F32: return transposeT<float>(in, xt, n, F, ld, stream);
    case DT_F64: return transposeT<double>(in, xt, n, F, ld, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t transposeInputsCoded(const float* in, float* xt, void* codes, int codeBytes, const int4* meta, size_t n, int F,
                                 size_t ld, cudaStream_t stream) {
  dim3 grid((unsigned)((ld + 31) / 32), (unsigned)((F + 31) / 32)), block(32, 8);
  if (codeBytes == 1) transposeCodedKernel<unsigned char><<<grid, block, 0, stream>>>(in, xt, (unsigned char*)codes, meta, n, F, ld);
  else transposeCodedKernel<unsigned short><<<grid, block, 0, stream>>>(in, xt, (unsigned short*)codes, meta, n, F, ld);
  return cudaGetLastError();
}

size_t layeredSmemBytes(const LayeredArgs& a, int tile) {
  return ((size_t)a.maxDepth * KMAX * tile + KMAX * KMAX) * 4 + (size_t)a.maxLeafFeatures * KMAX * 16;
}

cudaError_t layeredOccupancy(int tile, size_t smem, int* blocksPerSM) {
  cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&layeredKernel<float, true>), smem);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocksPerSM, layeredKernel<float, true>, tile, smem);
}

cudaError_t layeredLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid, int tile,
                          size_t smem, cudaStream_t stream) {
  switch (dtypeCode) {
    case DT_U8: return launchT<uint8_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_I8: return launchT<int8_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_U16: return launchT<uint16_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_I16: return launchT<int16_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_U32: return launchT<uint32_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_I32: return launchT<int32_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_U64: return launchT<uint64_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_I64: return launchT<int64_t>(a, in, out, n, grid, tile, smem, stream);
    case DT_F32: return launchT<float>(a, in, out, n, grid, tile, smem, stream);
    case DT_F64: return launchT<double>(a, in, out, n, grid, tile, smem, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace spnb
