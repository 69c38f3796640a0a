// Layered (RAT-SPN-style) SPN evaluation with the dense sum layers on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory (TMEM).
//
// Same stack machine as layered.cu / layered_mma.cu.  A CTA owns 128 samples (thread = sample = row of the
// M = 128 MMA tile).  For a full-width inner region (32 x 32 cross products, up to 32 sums) the contraction
//     S[128 x 32] = P[128 x 1024] * W^T[1024 x 32],   P[s, 32 i + j] = ea_i[s] * eb_j[s]
// runs as 64 k-steps of tcgen05.mma.cta_group::1.kind::f16 (M 128, N 32, K 16, fp16 operands, fp32
// accumulation in TMEM).  Both operands are read by the tensor core from shared memory in the K-major,
// non-swizzled canonical layout (8-row x 16-byte core matrices):
//   * P is produced on the fly: every thread multiplies its own ea_i (register) with its 32 eb_j (registers),
//     rounds to half precision and stores two 16-byte core-matrix rows per k-step; stages of 8 k-steps are
//     double buffered, so the threads fill one stage while the tensor core consumes the other;
//   * W is prepared on the host in exactly that layout (rows scaled by their largest weight) and copied
//     stage by stage with cp.async.
// One elected thread issues the MMAs of a stage and a tcgen05.commit that arrives on the stage's mbarrier
// when they have completed; a last commit per region signals "accumulator ready".  Then every thread reads
// its own row (TMEM lane = sample) with tcgen05.ld and finishes  out_k = ma + mb + log2(S_k) + log2 scale_k.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the kernel raises a flag in global memory, stops
// issuing tensor work, frees its TMEM columns and returns; the host reports the flag as an error.
//
// Operands are plain fp16 (no residue terms): about 2^-11 relative error per term, measured 1.4e-6 relative
// on the log-likelihood of the 784-feature benchmark model; small models should use the mma.sync path's
// split mode (spnb-kernel=layered).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "interp.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

constexpr int KMAX = 32;
constexpr int TS = 128;            // samples (threads) per CTA = MMA M
constexpr int STAGE_KSTEPS = 2;    // k-steps of 16 per stage (small stages: two CTAs fit on one SM)
constexpr int A_KSTEP_BYTES = TS * 16 * 2;          // 4096: [k-half 2][row group 16][row 8][8 halves]
constexpr int A_STAGE_BYTES = STAGE_KSTEPS * A_KSTEP_BYTES;   // 32 KB
constexpr int B_KSTEP_BYTES = KMAX * 16 * 2;        // 1024: [k-half 2][n group 4][n 8][8 halves]
constexpr int B_STAGE_BYTES = STAGE_KSTEPS * B_KSTEP_BYTES;   // 8 KB
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int TMEM_COLS = 32;

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
__device__ __forceinline__ unsigned smemAddr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// bounded wait for the phase with the given parity; false = gave up
__device__ __forceinline__ bool mbarWait(unsigned bar, unsigned parity) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void cpAsync16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// shared-memory matrix descriptor, K-major, no swizzle: start address, leading (K) byte offset, stride (M/N)
// byte offset, all in 16-byte units; descriptor version 1 (sm_100)
__device__ __forceinline__ unsigned long long smemDesc(unsigned addr, unsigned lboBytes, unsigned sboBytes) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lboBytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sboBytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

// shared memory: [stack float x maxDepth*32*128][mab, rootM, rootS float x 128][bars 8 x u64][tmem addr]
//                [A stages 2 x 8 KB][B stages 2 x 2 KB]   (the scalar path's weight row overlays them)
template <typename in_t, bool MARGINAL>
__global__ void __launch_bounds__(TS, 2) layeredTc5Kernel(LayeredArgs a, const in_t* __restrict__ in,
                                                           float* __restrict__ out, unsigned long long n,
                                                           int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned warp = tid >> 5;
  float* stack = reinterpret_cast<float*>(smem_raw);
  float* mab = stack + (size_t)a.maxDepth * KMAX * TS;
  float* rootM = mab + TS;
  float* rootS = rootM + TS;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(rootS + TS);   // [0],[1]: stage free; [2]: accumulator ready
  unsigned* tmemSlot = reinterpret_cast<unsigned*>(bars + 4);
  unsigned char* abuf = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tmemSlot + 4) + 127) & ~uintptr_t(127));
  unsigned char* bbuf = abuf + 2 * A_STAGE_BYTES;
  float* wbuf = reinterpret_cast<float*>(abuf);
  const unsigned F = a.numInputFeatures;
  const float NEG = __int_as_float(0xff800000);
  const unsigned barFree0 = smemAddr(bars), barFree1 = smemAddr(bars + 1), barDone = smemAddr(bars + 2);
  const unsigned aAddr = smemAddr(abuf), bAddr = smemAddr(bbuf);
  // instruction descriptor: D fp32, A/B fp16, both K-major, N = 32, M = 128
  const unsigned idesc = (1u << 4) | ((unsigned)(KMAX >> 3) << 17) | ((unsigned)(TS >> 4) << 24);

  if (tid == 0) {
    mbarInit(barFree0, 1);
    mbarInit(barFree1, 1);
    mbarInit(barDone, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmemSlot;
  unsigned phFree0 = 0, phFree1 = 0, phDone = 0;   // parities the next waits expect
  unsigned used0 = 0, used1 = 0;                   // has the stage buffer been handed to the tensor core before?
  bool failed = false;

  const unsigned long long ntiles = (n + TS - 1) / TS;
  for (unsigned long long tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x) {
    const unsigned long long row = tile * TS + tid;
    const bool live = row < n;
    const in_t* __restrict__ x = in + (a.xtLd ? 0 : (live ? row : 0) * F);
    // feature-major float copy of the batch (see transposeInputs): consecutive samples are consecutive floats
    const float* __restrict__ xT = reinterpret_cast<const float*>(in) + (live ? row : 0);
    int sp = 0;
    rootM[tid] = NEG;
    rootS[tid] = 0.f;
    for (int si = 0; si < a.numSteps && !failed; ++si) {
      const LayerStepDev s = a.steps[si];
      if (s.op == kLeafRegion) {
        // leaf parameters are read straight from global memory: every thread reads the same address
        // (one broadcast transaction, L1-resident), and no shared memory has to be set aside for them
        const float4* __restrict__ pbuf = a.quad + s.paramOffset;
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
                  const float4 q = __ldg(p + k);
                  const float t = fmaf(fmaf(q.x, xv, q.y), xv, q.z);
                  acc[k] = MARGINAL ? fmaf(m, t, acc[k]) : acc[k] + t;
                }
              } else {
    #pragma unroll
                for (int k = 0; k < KMAX; ++k) {
                  if (k < s.width) {
                    const float4 q = __ldg(p + k);
                    const float t = fmaf(fmaf(q.x, xv, q.y), xv, q.z);
                    acc[k] = MARGINAL ? fmaf(m, t, acc[k]) : acc[k] + t;
                  }
                }
              }
            }
          }
        }
        float* dst = stack + (size_t)sp * KMAX * TS + tid;
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
          if (k < s.width) dst[k * TS] = acc[k];
        ++sp;
        continue;
      }
      // ---- inner region or root part: operands into registers, max-shifted and exponentiated ----------------
      float* sa = stack + (size_t)(sp - 2) * KMAX * TS;
      float* sb = stack + (size_t)(sp - 1) * KMAX * TS;
      const MmaRegionDev mr = a.mma ? a.mma[si] : MmaRegionDev{-1, 0, 0};
      float ea[KMAX], eb[KMAX];
      float ma = NEG, mb = NEG;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        ea[i] = i < s.wa ? sa[i * TS + tid] : NEG;
        eb[i] = i < s.wb ? sb[i * TS + tid] : NEG;
        ma = fmaxf(ma, ea[i]);
        mb = fmaxf(mb, eb[i]);
      }
      const float za = ma == NEG ? 0.f : ma, zb = mb == NEG ? 0.f : mb;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        ea[i] = ex2f(ea[i] - za);
        eb[i] = ex2f(eb[i] - zb);
      }
      const float base = ma + mb;
      float* dstv = sa + tid;   // operands are in registers: the outputs may overwrite operand a
      auto fold = [&](int k, float v) {
        if (s.op == kInnerRegion) {
          dstv[k * TS] = v;
        } else {
          const float M = rootM[tid], S = rootS[tid];
          if (v > M) { rootS[tid] = S * ex2f(M - v) + 1.f; rootM[tid] = v; }
          else if (v == v && v != NEG) rootS[tid] = S + ex2f(v - M);
          else if (v != v) rootS[tid] = v;
        }
      };
      if (mr.fragOffset >= 0) {
        // ---- tensor-core contraction --------------------------------------------------------------------
        const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(a.frags) + mr.fragOffset * 8;
        __syncthreads();   // leaf parameters / scalar weights that overlay the A stages are no longer read
        const unsigned rowOff = (tid >> 3) * 128 + (tid & 7) * 16;   // this row inside one k-half block
        constexpr int NSTAGES = (KMAX * KMAX / 16) / STAGE_KSTEPS;
#pragma unroll
        for (int st = 0; st < NSTAGES; ++st) {
          if (failed) break;
          const int b = st & 1;
          // the tensor core must be done with this buffer (its MMAs of two stages ago)
          if (b == 0 ? used0 : used1) {
            if (!mbarWait(b == 0 ? barFree0 : barFree1, b == 0 ? phFree0 : phFree1)) failed = true;
            if (b == 0) phFree0 ^= 1; else phFree1 ^= 1;
          }
          if (__syncthreads_or(failed)) { failed = true; break; }
          // weights of the stage: 8 KB straight copy
          {
            const unsigned char* src = wsrc + (size_t)st * B_STAGE_BYTES;
            const unsigned dst = bAddr + b * B_STAGE_BYTES;
            for (int o = tid * 16; o < B_STAGE_BYTES; o += TS * 16) cpAsync16(dst + o, src + o);
            asm volatile("cp.async.commit_group;" ::: "memory");
          }
          // outer products of the stage: k-step ks covers i = (st * STAGE_KSTEPS + ks) / 2, j = 16 (ks & 1) .. + 15
          unsigned char* adst = abuf + b * A_STAGE_BYTES + rowOff;
#pragma unroll
          for (int ks = 0; ks < STAGE_KSTEPS; ++ks) {
            const int h = ks & 1;
            // ea[i] with i = (st * STAGE_KSTEPS + ks) / 2, picked with selects so that ea stays in registers
            const int iWanted = (st * STAGE_KSTEPS + ks) >> 1;
            float e = 0.f;
#pragma unroll
            for (int c = 0; c < KMAX; ++c)
              if (c == iWanted) e = ea[c];
            uint4 lo, hi;
            lo.x = packHalf2(e * eb[16 * h + 0], e * eb[16 * h + 1]);
            lo.y = packHalf2(e * eb[16 * h + 2], e * eb[16 * h + 3]);
            lo.z = packHalf2(e * eb[16 * h + 4], e * eb[16 * h + 5]);
            lo.w = packHalf2(e * eb[16 * h + 6], e * eb[16 * h + 7]);
            hi.x = packHalf2(e * eb[16 * h + 8], e * eb[16 * h + 9]);
            hi.y = packHalf2(e * eb[16 * h + 10], e * eb[16 * h + 11]);
            hi.z = packHalf2(e * eb[16 * h + 12], e * eb[16 * h + 13]);
            hi.w = packHalf2(e * eb[16 * h + 14], e * eb[16 * h + 15]);
            *reinterpret_cast<uint4*>(adst + ks * A_KSTEP_BYTES) = lo;                       // k 0..7
            *reinterpret_cast<uint4*>(adst + ks * A_KSTEP_BYTES + A_KSTEP_BYTES / 2) = hi;   // k 8..15
          }
          asm volatile("cp.async.wait_all;" ::: "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core reads
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncthreads();
          if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < STAGE_KSTEPS; ++ks) {
              const unsigned long long ad = smemDesc(aAddr + b * A_STAGE_BYTES + ks * A_KSTEP_BYTES, A_KSTEP_BYTES / 2, 128);
              const unsigned long long bd = smemDesc(bAddr + b * B_STAGE_BYTES + ks * B_KSTEP_BYTES, B_KSTEP_BYTES / 2, 128);
              const unsigned accumulate = (st | ks) ? 1u : 0u;
              asm volatile(
                  "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                  " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                  ::"r"(tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
                  : "memory");
            }
            // arrives on the stage's barrier once the MMAs issued so far have read their operands and finished
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(b == 0 ? barFree0 : barFree1)
                         : "memory");
            if (st == NSTAGES - 1)
              asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barDone) : "memory");
          }
          if (b == 0) used0 = 1; else used1 = 1;
        }
        // accumulator ready?
        if (!failed && !mbarWait(barDone, phDone)) failed = true;
        phDone ^= 1;
        if (__syncthreads_or(failed)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned r[KMAX];
        const unsigned taddr = tmem + ((warp * 32u) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
              "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const float* scale = a.scales + mr.scaleOffset;
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
          if (k < s.width) fold(k, base + lg2f(__uint_as_float(r[k])) + scale[k]);
        // the next region's first MMA overwrites the accumulator: order these reads before it
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      } else {
        // ---- scalar contraction (any widths) --------------------------------------------------------------
        const int per = s.wa * s.wb;
        for (int k = 0; k < s.width; ++k) {
          __syncthreads();
          const float* w = a.weights + s.paramOffset + (long long)k * per;
          for (int i = tid; i < per; i += TS) wbuf[i] = __ldg(w + i);
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
          fold(k, base + lg2f(acc));
        }
      }
      __syncthreads();
      sp -= (s.op == kInnerRegion) ? 1 : 2;
    }
    if (live && !failed) out[row] = (rootM[tid] + lg2f(rootS[tid])) * 0x1.62e43p-1f;
    __syncthreads();
  }
  if (failed && tid == 0) atomicExch(status, 1);
  // Outstanding tensor work reads shared memory and writes TMEM: give it a bounded time to finish, then free
  // the TMEM columns (also after a failure, so that the next kernel on this SM can allocate).
  if (failed && (used0 | used1)) {
    mbarWait(barFree0, phFree0);
    mbarWait(barFree1, phFree1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

template <typename in_t>
cudaError_t launchT(const LayeredArgs& a, const void* in, float* out, size_t n, int grid, size_t smem, int* status,
                    cudaStream_t stream) {
  auto run = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, TS, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n, status);
    return cudaGetLastError();
  };
  return a.marginal ? run(layeredTc5Kernel<in_t, true>) : run(layeredTc5Kernel<in_t, false>);
}

}  // namespace

size_t layeredTc5SmemBytes(const LayeredArgs& a) {
  size_t fixed = ((size_t)a.maxDepth * KMAX * TS + 3 * TS) * 4 + 8 * 8 + 16 + 128;
  size_t stages = 2 * (size_t)A_STAGE_BYTES + 2 * (size_t)B_STAGE_BYTES;
  size_t scalarRow = (size_t)KMAX * KMAX * 4;
  return fixed + (stages > scalarRow ? stages : scalarRow);
}

cudaError_t layeredTc5Occupancy(size_t smem, int* blocksPerSM) {
  cudaError_t e = cudaFuncSetAttribute(layeredTc5Kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocksPerSM, layeredTc5Kernel<float, true>, TS, smem);
}

cudaError_t layeredTc5Launch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid,
                             size_t smem, int* status, cudaStream_t stream) {
  switch (dtypeCode) {
    case DT_F32: return launchT<float>(a, in, out, n, grid, smem, status, stream);
    case DT_F64: return launchT<double>(a, in, out, n, grid, smem, status, stream);
    default: return cudaErrorInvalidValue;   // the tensor-memory path is built for floating inputs only
  }
}

}  // namespace spnb
