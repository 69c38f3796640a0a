// Layered (RAT-SPN-style) SPN evaluation with the dense sum layers on the tensor cores.
//
// Same stack machine over region outputs as the scalar kernel (layered.cu); the difference is the inner
// region  out_k = ma + mb + log2( sum_{i,j} W_k[i,j] * ea_i * eb_j ):  for a CTA tile of 256 samples this is
// a [256 x 1024] x [1024 x 32] contraction whose left operand, the outer products ea_i * eb_j, is never
// stored: every thread multiplies the eight entries of its A fragment in registers, rounds them to half
// precision and feeds mma.sync.m16n8k16 (fp16 operands, fp32 accumulators).  The weights are prepared on
// the host as B fragments in issue order, each sum's row divided by its largest weight so that they fill
// the fp16 range, and are streamed through shared memory with cp.async, double buffered, 16 k-steps at a
// time.  All operands lie in (0, 1] (they are max-shifted), so half precision costs about 2^-11 relative
// error per term, i.e. an absolute error below 1e-3 in the base-2 log of a sum.  In split mode (default)
// both operands also carry their rounding residue as a second half-precision number and three products
// are accumulated (hi*hi + lo*hi + hi*lo), which brings the error down to about 2^-21 per term.
//
// This is the warp-level mma path of the SM (it also runs on sm_100a); it stands in for a tcgen05/TMEM
// version, against which it will serve as the reference.  The scalar kernel checks both.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "interp.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

constexpr int KMAX = 32;
constexpr int TM = 256;            // samples (threads) per CTA
constexpr int CHUNK_KSTEPS = 16;   // k-steps of 16 per weight chunk

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
__device__ __forceinline__ unsigned packHalf2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cpAsync16(void* smemDst, const void* gmemSrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smemDst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmemSrc) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// shared memory: [stack float x maxDepth*32*256][mab, rootM, rootS float x 256 each][buf: two weight chunks /
// leaf parameters / scalar weight row]
template <typename in_t, bool MARGINAL, bool SPLIT>
__global__ void __launch_bounds__(TM, 1) layeredMmaKernel(LayeredArgs a, const in_t* __restrict__ in,
                                                           float* __restrict__ out, unsigned long long n, int bufBytes) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned lane = tid & 31, wbase = tid & ~31u;
  const unsigned g = lane >> 2, tig = lane & 3;
  float* stack = reinterpret_cast<float*>(smem_raw);
  float* mab = stack + (size_t)a.maxDepth * KMAX * TM;
  float* rootM = mab + TM;
  float* rootS = rootM + TM;
  unsigned char* buf = reinterpret_cast<unsigned char*>(rootS + TM);
  float* wbuf = reinterpret_cast<float*>(buf);
  float4* pbuf = reinterpret_cast<float4*>(buf);
  const unsigned F = a.numInputFeatures;
  const float NEG = __int_as_float(0xff800000);

  const unsigned long long ntiles = (n + TM - 1) / TM;
  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const unsigned long long row = tile * TM + tid;
    const bool live = row < n;
    const in_t* __restrict__ x = in + (a.xtLd ? 0 : (live ? row : 0) * F);
    // feature-major float copy of the batch (see transposeInputs): consecutive samples are consecutive floats
    const float* __restrict__ xT = reinterpret_cast<const float*>(in) + (live ? row : 0);
    int sp = 0;
    rootM[tid] = NEG;
    rootS[tid] = 0.f;
    for (int si = 0; si < a.numSteps; ++si) {
      const LayerStepDev s = a.steps[si];
      if (s.op == kLeafRegion) {
        const int cnt = s.numFeatures * s.width;
        __syncthreads();
        for (int i = tid; i < cnt; i += TM) pbuf[i] = a.leafParams[s.paramOffset + i];
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
              if (s.width == KMAX) {
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
        float* dst = stack + (size_t)sp * KMAX * TM + tid;
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
          if (k < s.width) dst[k * TM] = acc[k];
        ++sp;
        continue;
      }
      // ---- inner region or root part -------------------------------------------------------------------
      float* sa = stack + (size_t)(sp - 2) * KMAX * TM;   // operand a, then ea, then (inner) the outputs
      float* sb = stack + (size_t)(sp - 1) * KMAX * TM;   // operand b, then eb
      const MmaRegionDev mr = a.mma ? a.mma[si] : MmaRegionDev{-1, 0, 0};
      // phase A (thread = sample): max-shift and exponentiate both operands in place
      {
        float va[KMAX], vb[KMAX];
        float ma = NEG, mb = NEG;
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          va[i] = i < s.wa ? sa[i * TM + tid] : NEG;
          vb[i] = i < s.wb ? sb[i * TM + tid] : NEG;
          ma = fmaxf(ma, va[i]);
          mb = fmaxf(mb, vb[i]);
        }
        const float za = ma == NEG ? 0.f : ma, zb = mb == NEG ? 0.f : mb;
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          if (i < s.wa) sa[i * TM + tid] = ex2f(va[i] - za);
          if (i < s.wb) sb[i * TM + tid] = ex2f(vb[i] - zb);
        }
        mab[tid] = ma + mb;
      }
      __syncthreads();  // ea / eb visible; the shared buffer is free
      if (mr.fragOffset >= 0) {
        // ---- tensor-core contraction: wa = wb = 32, k index = i * 32 + j --------------------------------
        const int nt = mr.numTiles;
        // SPLIT: every fragment is followed by the fragment of the weights' rounding residues
        const int chunkBytes = CHUNK_KSTEPS * nt * 32 * 8 * (SPLIT ? 2 : 1);
        const unsigned char* gsrc = reinterpret_cast<const unsigned char*>(a.frags + mr.fragOffset);
        const int nchunks = (KMAX * KMAX / 16) / CHUNK_KSTEPS;
        auto fetch = [&](int c) {
          unsigned char* dst = buf + (size_t)(c & 1) * (bufBytes / 2);
          const unsigned char* src = gsrc + (size_t)c * chunkBytes;
          for (int o = tid * 16; o < chunkBytes; o += TM * 16) cpAsync16(dst + o, src + o);
          cpAsyncCommit();
        };
        fetch(0);
        // eb entries this thread's A fragments need: rows g and g+8 of both 16-sample halves of the warp
        float eb[2][2][8];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const unsigned col = wbase + 16 * mt + g + 8 * r;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j0 = 16 * h + 2 * tig;
              eb[mt][r][4 * h + 0] = sb[(j0 + 0) * TM + col];
              eb[mt][r][4 * h + 1] = sb[(j0 + 1) * TM + col];
              eb[mt][r][4 * h + 2] = sb[(j0 + 8) * TM + col];
              eb[mt][r][4 * h + 3] = sb[(j0 + 9) * TM + col];
            }
          }
        float acc[2][4][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[mt][t][q] = 0.f;
        for (int c = 0; c < nchunks; ++c) {
          if (c + 1 < nchunks) {
            fetch(c + 1);
            cpAsyncWait<1>();
          } else {
            cpAsyncWait<0>();
          }
          __syncthreads();
          const uint2* wf = reinterpret_cast<const uint2*>(buf + (size_t)(c & 1) * (bufBytes / 2));
#pragma unroll 2
          for (int ii = 0; ii < CHUNK_KSTEPS / 2; ++ii) {
            const int i = c * (CHUNK_KSTEPS / 2) + ii;
            float ea[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              ea[mt][0] = sa[i * TM + wbase + 16 * mt + g];
              ea[mt][1] = sa[i * TM + wbase + 16 * mt + g + 8];
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              unsigned af[2][4], al[2][4];
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int r = q & 1, cpair = q >> 1;   // register q: row g + 8r, columns 2tig + 8*cpair, +1
                  const float p0 = ea[mt][r] * eb[mt][r][4 * h + 2 * cpair + 0];
                  const float p1 = ea[mt][r] * eb[mt][r][4 * h + 2 * cpair + 1];
                  const __half2 hi = __floats2half2_rn(p0, p1);
                  af[mt][q] = *reinterpret_cast<const unsigned*>(&hi);
                  if (SPLIT) {   // what half precision dropped, again in half precision
                    const float2 back = __half22float2(hi);
                    al[mt][q] = packHalf2(p0 - back.x, p1 - back.y);
                  }
                }
              }
              const int ks = 2 * ii + h;
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if (t < nt) {
                  if (SPLIT) {
                    const uint4 bf = reinterpret_cast<const uint4*>(wf)[(ks * nt + t) * 32 + lane];
                    mma16816(acc[0][t], af[0], bf.x, bf.y);
                    mma16816(acc[1][t], af[1], bf.x, bf.y);
                    mma16816(acc[0][t], al[0], bf.x, bf.y);
                    mma16816(acc[1][t], al[1], bf.x, bf.y);
                    mma16816(acc[0][t], af[0], bf.z, bf.w);
                    mma16816(acc[1][t], af[1], bf.z, bf.w);
                  } else {
                    const uint2 bf = wf[(ks * nt + t) * 32 + lane];
                    mma16816(acc[0][t], af[0], bf.x, bf.y);
                    mma16816(acc[1][t], af[1], bf.x, bf.y);
                  }
                }
              }
            }
          }
          __syncthreads();  // every warp is done with this chunk before its buffer is refilled
        }
        // epilogue: this thread holds sums 8t + 2tig, +1 for rows g, g+8 of both halves
        const float* scale = a.scales + mr.scaleOffset;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const unsigned col = wbase + 16 * mt + g + 8 * r;
            const float base = mab[col];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (t < nt) {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const int k = 8 * t + 2 * tig + q;
                  if (k < s.width) {
                    const float v = base + lg2f(acc[mt][t][2 * r + q]) + scale[k];
                    if (s.op == kInnerRegion) {
                      sa[k * TM + col] = v;
                    } else {
                      const float M = rootM[col], S = rootS[col];
                      if (v > M) { rootS[col] = S * ex2f(M - v) + 1.f; rootM[col] = v; }
                      else if (v == v && v != NEG) rootS[col] = S + ex2f(v - M);
                      else if (v != v) rootS[col] = v;
                    }
                  }
                }
              }
            }
          }
      } else {
        // ---- scalar contraction (any widths), one sum at a time through the shared weight row ---------
        float ea[KMAX], eb[KMAX];
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          ea[i] = i < s.wa ? sa[i * TM + tid] : 0.f;
          eb[i] = i < s.wb ? sb[i * TM + tid] : 0.f;
        }
        const int per = s.wa * s.wb;
        const float base = mab[tid];
        for (int k = 0; k < s.width; ++k) {
          __syncthreads();
          const float* w = a.weights + s.paramOffset + (long long)k * per;
          for (int i = tid; i < per; i += TM) wbuf[i] = __ldg(w + i);
          __syncthreads();
          float acc = 0.f;
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
          const float v = base + lg2f(acc);
          if (s.op == kInnerRegion) {
            sa[k * TM + tid] = v;
          } else {
            const float M = rootM[tid], S = rootS[tid];
            if (v > M) { rootS[tid] = S * ex2f(M - v) + 1.f; rootM[tid] = v; }
            else if (v == v && v != NEG) rootS[tid] = S + ex2f(v - M);
            else if (v != v) rootS[tid] = v;
          }
        }
      }
      __syncthreads();  // outputs written by other lanes are visible to the sample's own thread
      sp -= (s.op == kInnerRegion) ? 1 : 2;
    }
    if (live) out[row] = (rootM[tid] + lg2f(rootS[tid])) * 0x1.62e43p-1f;
    __syncthreads();
  }
}

template <typename in_t>
cudaError_t launchT(const LayeredArgs& a, const void* in, float* out, size_t n, int grid, size_t smem, int bufBytes,
                    cudaStream_t stream) {
  auto run = [&](auto kernel) -> cudaError_t {
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(kernel), smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, TM, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n, bufBytes);
    return cudaGetLastError();
  };
  if (a.split) return a.marginal ? run(layeredMmaKernel<in_t, true, true>) : run(layeredMmaKernel<in_t, false, true>);
  return a.marginal ? run(layeredMmaKernel<in_t, true, false>) : run(layeredMmaKernel<in_t, false, false>);
}

int mmaBufBytes(const LayeredArgs& a) {
  int b = 2 * CHUNK_KSTEPS * 4 * 32 * 8 * (a.split ? 2 : 1);      // two chunks of full-width fragments
  b = b > a.maxLeafFeatures * KMAX * 16 ? b : a.maxLeafFeatures * KMAX * 16;
  b = b > KMAX * KMAX * 4 ? b : KMAX * KMAX * 4;
  return (b + 31) & ~31;
}

}  // namespace

size_t layeredMmaSmemBytes(const LayeredArgs& a) {
  return ((size_t)a.maxDepth * KMAX * TM + 3 * TM) * 4 + (size_t)mmaBufBytes(a);
}

cudaError_t layeredMmaOccupancy(size_t smem, int* blocksPerSM) {
  cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&layeredMmaKernel<float, true, true>), smem);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocksPerSM, layeredMmaKernel<float, true, true>, TM, smem);
}

cudaError_t layeredMmaLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid,
                             size_t smem, cudaStream_t stream) {
  const int bufBytes = mmaBufBytes(a);
  switch (dtypeCode) {
    case DT_F32: return launchT<float>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_F64: return launchT<double>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_U8: return launchT<uint8_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_I8: return launchT<int8_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_U16: return launchT<uint16_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_I16: return launchT<int16_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_U32: return launchT<uint32_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_I32: return launchT<int32_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_U64: return launchT<uint64_t>(a, in, out, n, grid, smem, bufBytes, stream);
    case DT_I64: return launchT<int64_t>(a, in, out, n, grid, smem, bufBytes, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace spnb
