// Layered (RAT-SPN-style) SPN evaluation with BOTH kinds of region on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), the CUDA cores keeping only the epilogues.
//
// Same stack machine as layered.cu.  A CTA owns 128 samples: thread = sample = row of the M = 128 MMA tile =
// TMEM lane.  All operands are half precision carried as (value, rounding residue) pairs, products
// accumulate in fp32, so every contraction keeps about 22 significant bits.
//
// Inner region (operands a, b of 32 values each, up to 32 sums).  With ea_i = 2^(a_i - max a) and
// eb_j = 2^(b_j - max b) the sum  S_k = sum_ij W_k[i,j] ea_i eb_j  is evaluated in two steps,
//     T[s, (k,i)] = sum_j eb_j[s] * W_k[i,j]          tensor core: [128 x 32] x [32 x 1024]
//     S_k[s]      = sum_i ea_i[s] * T[s, (k,i)]       CUDA cores: 32 FMAs per sum, T read from TMEM
// so the threads never form the 1024 cross products: they write eb once per region (64 halves: value and
// residue) and the tensor core does the 32-fold larger part.  The (k,i) columns are processed in blocks of
// 128 (six MMAs of M 128, N 128, K 16 per block: value x value, residue x value, value x residue), the blocks
// alternate between two TMEM accumulators, and the weights of block n+2 are copied (cp.async, four shared
// buffers) while block n is multiplied and block n-1 is folded.
//
// Leaf region (Gaussian leaves; the base-2 log density of feature f under component k is the quadratic
// a_fk x^2 + b_fk x + c_fk).  With x' = x - centre_f (centre chosen per feature on the host) the region is
//     out[s, k] = sum_f [x'^2, x', 1] . [a'_fk, b'_fk, c'_fk]
// which is a [128 x 8 F] x [8 F x 32] product: per feature the eight operand entries are
//     A: (sh, sl, sh, xh, xl, xh, 1, 1)      B: (ah, ah, al, bh, bh, bl, ch, cl)
// (h = half-precision value, l = residue).  A missing input (NaN, marginalised) writes eight zeros.  The
// threads build one 16-byte row per feature; stages of eight features are double buffered against the MMAs.
// An input whose |x'| does not fit half precision (>= 240, squared: overflow) makes its thread recompute its
// row of the region with plain FP32 arithmetic afterwards, so the result never depends on the range.
//
// Both operands are read by the tensor core from shared memory in the K-major, non-swizzled canonical layout
// (8-row x 16-byte core matrices); weights are prepared on the host in exactly that layout.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the kernel raises a flag in global memory, stops
// issuing tensor work, frees its TMEM columns and returns; the host reports the flag as an error.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "interp.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

constexpr int KMAX = 32;
constexpr int TS = 128;                        // samples (threads) per CTA = MMA M
constexpr int KSTEP_A = TS * 16 * 2;           // 4096 B: one 128 x 16 operand block [k-half 2][row group 16][row 8][8 halves]
constexpr int LEAF_STAGE_KSTEPS = 4;           // eight features per stage
constexpr int A_STAGE = LEAF_STAGE_KSTEPS * KSTEP_A;   // 16 KB; the inner regions' operand (4 k-steps) uses stage 0
constexpr int A_BYTES = 2 * A_STAGE;
constexpr int NBLK = 128;                      // (k,i) columns per block of an inner region
constexpr int KSTEP_B = NBLK * 16 * 2;         // 4096 B
constexpr int B_BLOCK = 4 * KSTEP_B;           // value j 0..15, value j 16..31, residue j 0..15, residue j 16..31
constexpr int NBBUF = 4;                       // weight blocks are copied two blocks ahead of their MMAs
constexpr int B_BYTES = NBBUF * B_BLOCK;       // 64 KB
constexpr int KSTEP_BL = KMAX * 16 * 2;        // 1024 B: leaf weights of one k-step (two features)
constexpr int BL_STAGE = LEAF_STAGE_KSTEPS * KSTEP_BL;   // 4 KB; a ring of four stages at the start of the B area
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int TMEM_COLS = 512;                 // 2 x 128 inner accumulators, 32 leaf accumulator columns at 256
constexpr int TMEM_LEAF = 256;
constexpr int LEAF_Q = 4;                      // leaf stages the input queue runs ahead (a multiple of 4: ring slots are static)
constexpr float kHalfRange = 240.f;            // |x'| below this: x'^2 < 65504

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
// v as half-precision value (returned as float) and the residue v - value
__device__ __forceinline__ void splitHalf(float v, float& hi, float& lo) {
  hi = __half2float(__float2half_rn(v));
  lo = v - hi;
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
__device__ __forceinline__ void mbarArrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cpAsync16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void mmaF16(unsigned d, unsigned long long ad, unsigned long long bd, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d),
      "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void mmaCommit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// this thread's N consecutive accumulator columns (lane = its sample), N = 8, 16 or 32
__device__ __forceinline__ void tmemLoad8(unsigned taddr, unsigned* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemLoad16(unsigned taddr, unsigned* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemLoad32(unsigned taddr, unsigned* r) {
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
}

// shared-memory matrix descriptor, K-major, no swizzle: start address, leading (K) byte offset, stride (M/N)
// byte offset, all in 16-byte units; descriptor version 1 (sm_100)
__device__ __forceinline__ unsigned long long smemDesc(unsigned addr, unsigned lboBytes, unsigned sboBytes) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lboBytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sboBytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

// shared memory: [stack float x maxDepth*32*128][rootM, rootS float x 128][redo flags int x 2 x 128]
//                [bars 16 x u64][tmem addr][A: 2 x 16 KB][B: 4 x 16 KB]   (the scalar contraction's weight row
//                overlays A)
//
// The CTA has NWG warpgroups of 128 worker threads plus one warp that only issues tensor-core work.  Worker
// t works on sample t % 128; the warpgroups split the work of every region between them (features of a leaf
// stage, operand columns, sums of a block).  Workers and the issuing warp meet only through mbarriers inside
// a region:  workers arrive on a "ready" barrier when their part of the operands is in shared memory (and the
// accumulator they are about to overwrite has been read); the issuing warp waits for it, issues the MMAs and
// commits them to a "done" barrier that the workers wait for before they read the accumulator or reuse the
// operand buffer.  CTA-wide barriers remain only at the region boundaries.
template <typename in_t, bool MARGINAL, int NWG>
__global__ void __launch_bounds__(TS * NWG + 32, 1) layeredTcfKernel(LayeredArgs a, const in_t* __restrict__ in,
                                                                     float* __restrict__ out, unsigned long long n,
                                                                     int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int NT = TS * NWG;            // worker threads
  const unsigned tid = threadIdx.x;
  const unsigned warp = tid >> 5;
  const bool issuer = tid >= NT;          // the last warp
  const unsigned r128 = tid & (TS - 1);   // the sample (row) inside the tile
  const unsigned wg = issuer ? 0 : tid >> 7;
  float* stack = reinterpret_cast<float*>(smem_raw);
  float* rootM = stack + (size_t)a.maxDepth * KMAX * TS;
  float* rootS = rootM + TS;
  int* redoFlag = reinterpret_cast<int*>(rootS + TS);   // [2][128]: an input of the leaf region was out of range
  // mbarriers.  Issuer -> workers ("done", count 1, tcgen05.commit arrives):
  //   [0],[1] leaf stage buffer consumed; [2] leaf accumulator ready; [3],[4] inner block in accumulator 0 / 1 ready
  // Workers -> issuer ("ready", count NT):
  //   [5],[6] leaf stage buffer filled; [7],[8] inner block operands in place and accumulator 0 / 1 free
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(redoFlag + 2 * TS);
  unsigned* tmemSlot = reinterpret_cast<unsigned*>(bars + 12);
  unsigned char* abuf = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(tmemSlot + 4) + 127) & ~uintptr_t(127));
  unsigned char* bbuf = abuf + A_BYTES;
  float* wbuf = reinterpret_cast<float*>(abuf);
  const unsigned F = a.numInputFeatures;
  const float NEG = __int_as_float(0xff800000);
  const unsigned barStage0 = smemAddr(bars), barStage1 = smemAddr(bars + 1), barLeaf = smemAddr(bars + 2);
  const unsigned barBlk0 = smemAddr(bars + 3), barBlk1 = smemAddr(bars + 4);
  const unsigned barFull0 = smemAddr(bars + 5), barFull1 = smemAddr(bars + 6);
  const unsigned barReady0 = smemAddr(bars + 7), barReady1 = smemAddr(bars + 8);
  const unsigned aAddr = smemAddr(abuf), bAddr = smemAddr(bbuf);
  // instruction descriptors: D fp32, A/B fp16, both K-major, M = 128, N = 32 (leaf) / 128 (inner)
  const unsigned idescLeaf = (1u << 4) | ((unsigned)(KMAX >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
  const unsigned idescSum = (1u << 4) | ((unsigned)(NBLK >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
  // descriptors of the operand areas' first blocks; a block further on adds its byte offset / 16 to the
  // start-address field (the sum stays inside the field: shared memory ends below 256 KB)
  const unsigned long long aDesc0 = smemDesc(aAddr, KSTEP_A / 2, 128);
  const unsigned long long bDesc0 = smemDesc(bAddr, KSTEP_B / 2, 128);
  const unsigned long long blDesc0 = smemDesc(bAddr, KSTEP_BL / 2, 128);
  const unsigned rowOff = (r128 >> 3) * 128 + (r128 & 7) * 16;   // this thread's row inside one k-half block

  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbarInit(smemAddr(bars + i), 1);
    for (int i = 5; i < 9; ++i) mbarInit(smemAddr(bars + i), NT);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 2 * TS) redoFlag[tid] = 0;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmemSlot;
  const unsigned tmemLane = tmem + (((warp & 3u) * 32u) << 16);   // a warp reaches the lane quarter warp % 4
  // parities the next waits expect.  Workers wait on the "done" barriers, the issuer on the "ready" ones.
  unsigned phStage0 = 0, phStage1 = 0, phLeaf = 0, phBlk0 = 0, phBlk1 = 0;
  unsigned phFull0 = 0, phFull1 = 0, phReady0 = 0, phReady1 = 0;
  unsigned pend0 = 0, pend1 = 0;   // a leaf stage commit on barStage0 / 1 has not been waited for yet
  unsigned pendBlk0 = 0, pendBlk1 = 0, pendLeaf = 0;
  unsigned leafParity = 0;
  bool failed = false;

  const unsigned long long ntiles = (n + TS - 1) / TS;
  for (unsigned long long tile = blockIdx.x; tile < ntiles && !failed; tile += gridDim.x) {
    const unsigned long long row = tile * TS + r128;
    const bool live = row < n;
    const in_t* __restrict__ x = in + (a.xtLd ? 0 : (live ? row : 0) * F);
    // feature-major float copy of the batch (see transposeInputs): consecutive samples are consecutive floats
    const float* __restrict__ xT = reinterpret_cast<const float*>(in) + (live ? row : 0);
    constexpr int FPW = 8 / NWG;      // features of a leaf stage per warpgroup
    float xq[LEAF_Q][FPW], cq[LEAF_Q][FPW];
    auto loadSlot = [&](int d, int g) {
      g = g < a.numLeafStages ? g : a.numLeafStages - 1;
#pragma unroll
      for (int u = 0; u < FPW; ++u) {
        const int at = g * 8 + wg * FPW + u;
        const int col = __ldg(a.leafCols + at);   // padding entries name column 0
        xq[d][u] = a.xtLd ? xT[(size_t)col * a.xtLd] : (float)x[col];
        cq[d][u] = __ldg(a.leafCentres + at);
      }
    };
    if (a.numLeafStages > 0 && !issuer) {
#pragma unroll
      for (int d = 0; d < LEAF_Q; ++d) loadSlot(d, d);
    } else {
#pragma unroll
      for (int d = 0; d < LEAF_Q; ++d)
#pragma unroll
        for (int u = 0; u < FPW; ++u) xq[d][u] = cq[d][u] = 0.f;
    }
    int sp = 0;
    if (tid < TS) {
      rootM[r128] = NEG;
      rootS[r128] = 0.f;
    }
    for (int si = 0; si < a.numSteps && !failed; ++si) {
      const LayerStepDev s = a.steps[si];
      const MmaRegionDev mr = a.mma[si];
      if (s.op == kLeafRegion) {
        constexpr int KPW = KMAX / NWG;   // outputs per warpgroup
        unsigned r[KPW];
        bool redo = mr.fragOffset < 0;    // regions without tensor-core weights are computed by the FP32 loop below
        if (mr.fragOffset >= 0) {
          const int nst = (s.numFeatures + 7) >> 3;
          if (issuer) {
            // ---- issuing warp: one batch of MMAs per stage, as soon as the workers have filled it ------------
#pragma unroll 1
            for (int st = 0; st < nst && !failed; ++st) {
              const int b = st & 1;
              if (!mbarWait(b == 0 ? barFull0 : barFull1, b == 0 ? phFull0 : phFull1)) failed = true;
              if (b == 0) phFull0 ^= 1; else phFull1 ^= 1;
              if (!failed && tid == NT) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < LEAF_STAGE_KSTEPS; ++ks) {
                  const unsigned long long ad = aDesc0 + (unsigned)((b * A_STAGE + ks * KSTEP_A) >> 4);
                  const unsigned long long bd = blDesc0 + (unsigned)(((st & 3) * BL_STAGE + ks * KSTEP_BL) >> 4);
                  mmaF16(tmem + TMEM_LEAF, ad, bd, idescLeaf, (st | ks) ? 1u : 0u);
                }
                mmaCommit(b == 0 ? barStage0 : barStage1);
                if (st == nst - 1) mmaCommit(barLeaf);
              }
              __syncwarp();
            }
          } else {
            // ---- workers ------------------------------------------------------------------------------------
            const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(a.frags) + mr.fragOffset * 8;
            // weights of stage st go to ring slot st % 4, two stages ahead of their MMAs; a group is committed
            // for every stage (empty past the end), so that the waits below can count groups
            auto copyStage = [&](int st) {
              if (st < nst) {
                const unsigned char* src = wsrc + (size_t)st * BL_STAGE;
                const unsigned dst = bAddr + (st & 3) * BL_STAGE;
                for (int o = tid * 16; o < BL_STAGE; o += NT * 16) cpAsync16(dst + o, src + o);
              }
              asm volatile("cp.async.commit_group;" ::: "memory");
            };
            copyStage(0);
            copyStage(1);
            // Inputs come through a register queue that runs LEAF_Q stages ahead of their use and carries on
            // across regions: the host lists the stages of all tensor-core leaf regions in execution order,
            // every region padded to a multiple of LEAF_Q stages, so stage st of a region always sits in queue
            // slot st % LEAF_Q.  A slot is refilled right after it has been consumed.
            const int gBase = mr.scaleOffset;
            const int nstPad = (nst + LEAF_Q - 1) / LEAF_Q * LEAF_Q;
            int* myRedo = redoFlag + leafParity * TS + r128;
#pragma unroll 1
            for (int st0 = 0; st0 < nstPad; st0 += LEAF_Q) {
#pragma unroll
              for (int d = 0; d < LEAF_Q; ++d) {
                const int st = st0 + d;
                if (st < nst && !failed) {
                  const int b = d & 1;
                  // the tensor core must be done with this stage buffer (its MMAs of two stages ago); the weight
                  // ring slot of stage st + 2 was read by the same MMAs
                  if (b == 0 ? pend0 : pend1) {
                    if (!mbarWait(b == 0 ? barStage0 : barStage1, b == 0 ? phStage0 : phStage1)) failed = true;
                    if (b == 0) { phStage0 ^= 1; pend0 = 0; } else { phStage1 ^= 1; pend1 = 0; }
                  }
                  if (!failed) {
                    copyStage(st + 2);
                    unsigned char* adst = abuf + b * A_STAGE + rowOff;
#pragma unroll
                    for (int u = 0; u < FPW; ++u) {
                      const int u8 = wg * FPW + u;   // position inside the stage
                      const int f = st * 8 + u8;
                      const float xv = xq[d][u];
                      const bool inRegion = f < s.numFeatures;
                      const bool valid = inRegion && (!MARGINAL || xv == xv);
                      const float xp = xv - cq[d][u];
                      if (valid && !(fabsf(xp) < kHalfRange)) *myRedo = 1;
                      float xh, xl, sh, sl;
                      splitHalf(xp, xh, xl);
                      splitHalf(xp * xp, sh, sl);
                      uint4 w;
                      w.x = packHalf2(sh, sl);
                      w.y = packHalf2(sh, xh);
                      w.z = packHalf2(xl, xh);
                      w.w = 0x3C003C00u;   // (1, 1)
                      if (!valid) w = make_uint4(0u, 0u, 0u, 0u);
                      // feature 2 t of the stage is k 0..7 of k-step t, feature 2 t + 1 is k 8..15
                      *reinterpret_cast<uint4*>(adst + (u8 >> 1) * KSTEP_A + (u8 & 1) * (KSTEP_A / 2)) = w;
                    }
                    asm volatile("cp.async.wait_group 2;" ::: "memory");   // all but the two newest groups: stage st has landed
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core reads
                    mbarArrive(b == 0 ? barFull0 : barFull1);
                    if (b == 0) pend0 = 1; else pend1 = 1;
                    if (st == nst - 1) pendLeaf = 1;
                  }
                }
                loadSlot(d, gBase + st + LEAF_Q);
              }
            }
            // accumulator ready; the stage barriers' last completions are consumed here as well, so that the
            // buffers are known to be free when the next region starts
            if (!failed && pendLeaf) { if (!mbarWait(barLeaf, phLeaf)) failed = true; phLeaf ^= 1; pendLeaf = 0; }
            if (!failed && pend0) { if (!mbarWait(barStage0, phStage0)) failed = true; phStage0 ^= 1; pend0 = 0; }
            if (!failed && pend1) { if (!mbarWait(barStage1, phStage1)) failed = true; phStage1 ^= 1; pend1 = 0; }
          }
          if (__syncthreads_or(failed)) { failed = true; break; }
          if (!issuer) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (redoFlag[leafParity * TS + r128]) redo = true;
            if constexpr (KPW == 32) tmemLoad32(tmemLane + TMEM_LEAF, r);
            else if constexpr (KPW == 16) tmemLoad16(tmemLane + TMEM_LEAF + wg * KPW, r);
            else tmemLoad8(tmemLane + TMEM_LEAF + wg * KPW, r);
            // the next leaf region's first MMA overwrites the accumulator: order these reads before it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // the other parity's flag was read in the previous leaf region, two CTA barriers ago
            if (wg == 0) redoFlag[(leafParity ^ 1) * TS + r128] = 0;
          }
          leafParity ^= 1;
        }
        if (redo && !issuer) {
          // plain FP32 evaluation of this thread's share of the row (out-of-range input, or a region without
          // tensor weights)
#pragma unroll
          for (int k = 0; k < KPW; ++k) r[k] = 0u;
          const float4* __restrict__ pbuf = a.leafParams + s.paramOffset;
          for (int f = 0; f < s.numFeatures; ++f) {
            const int col = __ldg(a.features + s.featOffset + f);
            float xv = a.xtLd ? xT[(size_t)col * a.xtLd] : (float)x[col];
            float m = 1.f;
            if (MARGINAL && xv != xv) { xv = 0.f; m = 0.f; }
            const float4* p = pbuf + f * s.width + wg * KPW;
#pragma unroll
            for (int k = 0; k < KPW; ++k) {
              if (wg * KPW + k < s.width) {
                const float4 q = __ldg(p + k);
                const float dx = xv - q.x;
                const float t = fmaf(dx * dx, q.y, q.z);
                const float acc = __uint_as_float(r[k]);
                r[k] = __float_as_uint(MARGINAL ? fmaf(m, t, acc) : acc + t);
              }
            }
          }
        }
        if (!issuer) {
          float* dst = stack + ((size_t)sp * KMAX + wg * KPW) * TS + r128;
#pragma unroll
          for (int k = 0; k < KPW; ++k)
            if (wg * KPW + k < s.width) dst[k * TS] = __uint_as_float(r[k]);
        }
        ++sp;
        __syncthreads();   // the other warpgroups read these values in the next step
        continue;
      }
      // ---- inner region or root part ------------------------------------------------------------------------
      const bool tensor = mr.fragOffset >= 0;
      if (issuer) {
        if (tensor) {
          const int nblk = mr.numTiles;
#pragma unroll 1
          for (int nb = 0; nb < nblk && !failed; ++nb) {
            const int b = nb & 1;
            if (!mbarWait(b == 0 ? barReady0 : barReady1, b == 0 ? phReady0 : phReady1)) failed = true;
            if (b == 0) phReady0 ^= 1; else phReady1 ^= 1;
            if (!failed && tid == NT) {
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              const unsigned long long bb = bDesc0 + (unsigned)(((nb % NBBUF) * B_BLOCK) >> 4);
              const unsigned d = tmem + b * NBLK;
              // value x value, residue x value, value x residue, each over j 0..15 and j 16..31
#pragma unroll
              for (int m = 0; m < 6; ++m) {
                const int aks = (m < 4) ? m : m - 4;   // A k-step: 0,1 value; 2,3 residue; 0,1 value
                const int bks = (m < 2) ? m : m - 2;   // B k-step: 0,1 value; 0,1 value; 2,3 residue
                const unsigned long long ad = aDesc0 + (unsigned)((aks * KSTEP_A) >> 4);
                const unsigned long long bd = bb + (unsigned)((bks * KSTEP_B) >> 4);
                mmaF16(d, ad, bd, idescSum, m ? 1u : 0u);
              }
              mmaCommit(b == 0 ? barBlk0 : barBlk1);
            }
            __syncwarp();
          }
        } else {
          for (int k = 0; k < s.width; ++k) {   // the scalar contraction's CTA barriers
            __syncthreads();
            __syncthreads();
          }
        }
        failed = __syncthreads_or(failed);
        sp -= (s.op == kInnerRegion) ? 1 : 2;
        continue;
      }
      const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(a.frags) + (tensor ? mr.fragOffset : 0) * 8;
      // a group is committed for every block (empty past the end), so that the waits can count groups
      auto copyBlock = [&](int nb) {
        if (nb < mr.numTiles) {
          const unsigned char* src = wsrc + (size_t)nb * B_BLOCK;
          const unsigned dst = bAddr + (nb % NBBUF) * B_BLOCK;
          for (int o = tid * 16; o < B_BLOCK; o += NT * 16) cpAsync16(dst + o, src + o);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
      // the first two blocks of weights travel while the operands are prepared (every earlier MMA has completed)
      if (tensor) {
        copyBlock(0);
        copyBlock(1);
      }
      float* sa = stack + (size_t)(sp - 2) * KMAX * TS;
      float* sb = stack + (size_t)(sp - 1) * KMAX * TS;
      constexpr int JPW = KMAX / NWG;   // columns j of operand b this warpgroup writes for the tensor core
      float ea[KMAX], eb[KMAX];
      float ma = NEG, mb = NEG;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        ea[i] = i < s.wa ? sa[i * TS + r128] : NEG;
        eb[i] = i < s.wb ? sb[i * TS + r128] : NEG;
        ma = fmaxf(ma, ea[i]);
        mb = fmaxf(mb, eb[i]);
      }
      const float za = ma == NEG ? 0.f : ma, zb = mb == NEG ? 0.f : mb;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) ea[i] = ex2f(ea[i] - za);
      if (tensor) {
        // only this warpgroup's share of operand b is needed in linear space
#pragma unroll
        for (int g = 0; g < KMAX / JPW; ++g)
          if (g == (int)wg) {
#pragma unroll
            for (int j = 0; j < JPW; ++j) eb[g * JPW + j] = ex2f(eb[g * JPW + j] - zb);
          }
      } else {
#pragma unroll
        for (int i = 0; i < KMAX; ++i) eb[i] = ex2f(eb[i] - zb);
      }
      const float base = ma + mb;
      // The outputs overwrite operand a's stack entry.  The first of them is written after the first block's
      // MMAs have completed, which were issued after every worker had read its operands and arrived.
      float* dstv = sa + r128;
      auto fold = [&](int k, float v) {
        if (s.op == kInnerRegion) {
          dstv[k * TS] = v;
        } else {
          const float M = rootM[r128], S = rootS[r128];
          if (v > M) { rootS[r128] = S * ex2f(M - v) + 1.f; rootM[r128] = v; }
          else if (v == v && v != NEG) rootS[r128] = S + ex2f(v - M);
          else if (v != v) rootS[r128] = v;
        }
      };
      if (tensor) {
        // operand A: k-steps 0, 1 = value of eb_j (j 0..15, 16..31), k-steps 2, 3 = residue
        {
          unsigned char* adst = abuf + rowOff;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int kh = 0; kh < 2; ++kh) {
              if ((16 * h + 8 * kh) / JPW != (int)wg) continue;   // another warpgroup's columns
              float vh[8], vl[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) splitHalf(eb[16 * h + 8 * kh + q], vh[q], vl[q]);
              uint4 hi, lo;
              hi.x = packHalf2(vh[0], vh[1]); hi.y = packHalf2(vh[2], vh[3]);
              hi.z = packHalf2(vh[4], vh[5]); hi.w = packHalf2(vh[6], vh[7]);
              lo.x = packHalf2(vl[0], vl[1]); lo.y = packHalf2(vl[2], vl[3]);
              lo.z = packHalf2(vl[4], vl[5]); lo.w = packHalf2(vl[6], vl[7]);
              *reinterpret_cast<uint4*>(adst + h * KSTEP_A + kh * (KSTEP_A / 2)) = hi;
              *reinterpret_cast<uint4*>(adst + (2 + h) * KSTEP_A + kh * (KSTEP_A / 2)) = lo;
            }
          }
        }
        const float* scale = a.scales + mr.scaleOffset;
        const int nblk = mr.numTiles;
        // fold block `blk` (sums 4 blk .. 4 blk + 3): wait for its MMAs, read T from TMEM, dot with ea
        auto epilogue = [&](int blk) {
          const int b = blk & 1;
          constexpr int KKPW = (NBLK / KMAX) / NWG;   // sums of a block per warpgroup
          float sc[KKPW];
#pragma unroll
          for (int q = 0; q < KKPW; ++q) {   // requested before the wait, used after it
            const int k = (NBLK / KMAX) * blk + wg * KKPW + q;
            sc[q] = __ldg(scale + (k < KMAX ? k : KMAX - 1));
          }
          if (!failed) {
            if (!mbarWait(b == 0 ? barBlk0 : barBlk1, b == 0 ? phBlk0 : phBlk1)) failed = true;
            if (b == 0) { phBlk0 ^= 1; pendBlk0 = 0; } else { phBlk1 ^= 1; pendBlk1 = 0; }
          }
          if (failed) return;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int q = 0; q < KKPW; ++q) {
            const int kk = wg * KKPW + q;
            const int k = (NBLK / KMAX) * blk + kk;
            if (k < s.width) {
              unsigned t[KMAX];
              tmemLoad32(tmemLane + b * NBLK + kk * KMAX, t);
              float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
              for (int i = 0; i < KMAX; i += 4) {
                acc0 = fmaf(ea[i], __uint_as_float(t[i]), acc0);
                acc1 = fmaf(ea[i + 1], __uint_as_float(t[i + 1]), acc1);
                acc2 = fmaf(ea[i + 2], __uint_as_float(t[i + 2]), acc2);
                acc3 = fmaf(ea[i + 3], __uint_as_float(t[i + 3]), acc3);
              }
              fold(k, base + lg2f((acc0 + acc1) + (acc2 + acc3)) + sc[q]);
            }
          }
          // a later block's MMAs overwrite this accumulator: order these reads before the arrival that allows them
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        };
#pragma unroll 1
        for (int nb = 0; nb < nblk && !failed; ++nb) {
          const int b = nb & 1;
          // this thread's part of block nb's weights has landed (all but the newest group), its part of operand
          // A is written (nb = 0) and it has read accumulator b for the last time (epilogue of block nb - 2)
          asm volatile("cp.async.wait_group 1;" ::: "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbarArrive(b == 0 ? barReady0 : barReady1);
          if (b == 0) pendBlk0 = 1; else pendBlk1 = 1;
          // weights of the block after the next: their buffer was last read by block nb - 2, whose completion
          // this thread has waited for in that block's epilogue
          copyBlock(nb + 2);
          if (nb >= 1) epilogue(nb - 1);
        }
        if (nblk > 0) epilogue(nblk - 1);
      } else {
        // ---- scalar contraction (any widths) --------------------------------------------------------------
        const int per = s.wa * s.wb;
        for (int k = 0; k < s.width; ++k) {
          __syncthreads();
          const float* w = a.weights + s.paramOffset + (long long)k * per;
          for (int i = tid; i < per; i += NT) wbuf[i] = __ldg(w + i);
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
          if (k % NWG == (int)wg) fold(k, base + lg2f(acc));   // every warpgroup computes it, one stores it
        }
      }
      failed = __syncthreads_or(failed);
      sp -= (s.op == kInnerRegion) ? 1 : 2;
    }
    if (tid < TS && live && !failed) out[row] = (rootM[r128] + lg2f(rootS[r128])) * 0x1.62e43p-1f;
    failed = __syncthreads_or(failed);
  }
  failed = __syncthreads_or(failed);
  if (failed && tid == 0) atomicExch(status, 1);
  // Outstanding tensor work reads shared memory and writes TMEM: give it a bounded time to finish, then free
  // the TMEM columns (also after a failure, so that the next kernel on this SM can allocate).
  if (failed && !issuer) {
    if (pend0) mbarWait(barStage0, phStage0);
    if (pend1) mbarWait(barStage1, phStage1);
    if (pendLeaf) mbarWait(barLeaf, phLeaf);
    if (pendBlk0) mbarWait(barBlk0, phBlk0);
    if (pendBlk1) mbarWait(barBlk1, phBlk1);
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
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
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(kernel), smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, TS * a.warpgroups + 32, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n, status);
    return cudaGetLastError();
  };
  switch (a.warpgroups) {
    case 1: return a.marginal ? run(layeredTcfKernel<in_t, true, 1>) : run(layeredTcfKernel<in_t, false, 1>);
    case 2: return a.marginal ? run(layeredTcfKernel<in_t, true, 2>) : run(layeredTcfKernel<in_t, false, 2>);
    case 4: return a.marginal ? run(layeredTcfKernel<in_t, true, 4>) : run(layeredTcfKernel<in_t, false, 4>);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// The kernel allocates all 512 TMEM columns of its SM, so two of its CTAs must never share an SM: the
// shared-memory request is kept above half of an SM's capacity.
size_t layeredTcfSmemBytes(const LayeredArgs& a) {
  size_t fixed = ((size_t)a.maxDepth * KMAX * TS + 4 * TS) * 4 + 12 * 8 + 16 + 128;
  size_t total = fixed + A_BYTES + B_BYTES;
  const size_t floor = 120 * 1024;
  return total > floor ? total : floor;
}

cudaError_t layeredTcfLaunch(const LayeredArgs& a, int dtypeCode, const void* in, float* out, size_t n, int grid,
                             size_t smem, int* status, cudaStream_t stream) {
  switch (dtypeCode) {
    case DT_F32: return launchT<float>(a, in, out, n, grid, smem, status, stream);
    case DT_F64: return launchT<double>(a, in, out, n, grid, smem, status, stream);
    default: return cudaErrorInvalidValue;   // the tensor-memory path is built for floating inputs only
  }
}

}  // namespace spnb
