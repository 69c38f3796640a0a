// Layered (RAT-SPN-style) SPN evaluation on the 5th-generation tensor cores, two sample tiles per CTA.
//
// Same arithmetic as layered_tcf.cu (factorised inner regions T = eb x W on tcgen05.mma with TMEM accumulators,
// S_k = sum_i ea_i T[(k,i)] on the CUDA cores; leaf regions as [x'^2, x', 1] x parameters, all operands half
// precision carried as value + rounding residue), but scheduled so that the tensor pipe does not wait for
// one tile's dependency chain:
//
//   * A CTA owns TWO tiles of 128 samples.  Both walk the same region program in lock step, so every block of
//     weights that is brought into shared memory is used by two MMAs groups (half the L2 -> shared traffic per
//     sample), and while the threads of one tile fold an accumulator the tensor core works for the other.
//   * Warp roles: warps 0-3 = tile 0, warps 4-7 = tile 1 (thread = sample = TMEM lane), warp 8 issues every
//     MMA, warp 9 streams inner-region weights and warp 10 leaf weights with bulk asynchronous copies
//     (cp.async.bulk global -> shared, completion counted on an mbarrier; no multicast).  Roles meet only
//     through mbarriers; there is no CTA-wide barrier inside the tile loop.
//   * Region outputs no longer go through a five-deep stack in shared memory.  In the post-order walk the
//     right operand (b) of a region is always produced by the step directly before it: its producer writes
//     it straight into the tile's MMA operand buffer (2^(b - max b) as value / residue halves).  Left
//     operands (a) wait in a small "a-stack" (one 16 KB slot per pending left operand), or stay in registers
//     when the right sibling is a single leaf region.  Leaf accumulators are read from TMEM by their consumer.
//   * TMEM: 512 columns = 2 tiles x 2 accumulators x 128 columns; a leaf region uses the first 32 columns of
//     its tile's accumulator 0.
//
// Every mbarrier wait is bounded.  A wait that runs out raises a CTA-wide abort flag (all roles poll it) and
// the status word in global memory; the CTA then waits, again bounded, for its outstanding copies and MMAs,
// frees its TMEM columns and returns.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstdlib>

#include "interp.h"
#include "layered.h"
#include "layers.h"

namespace spnb {

namespace {

constexpr int KMAX = 32;
constexpr int TS = 128;                 // samples per tile = MMA M
constexpr int NTILE = 2;                // tiles per CTA
constexpr int NWORK = NTILE * TS;       // worker threads
constexpr int NTHREADS = NWORK + 96;    // + issuer warp, weight loader warp, leaf-weight loader warp
constexpr int KSTEP_A = TS * 16 * 2;    // 4096 B: one 128 x 16 operand block [k-half 2][row group 16][row 8][8 halves]
constexpr int A_TILE = 4 * KSTEP_A;     // 16 KB per tile: inner operand (4 k-steps) or two leaf stages of 2 k-steps
constexpr int LEAF_STAGE = 2 * KSTEP_A; // 8 KB: four features
constexpr int NBLK = 128;               // (k,i) columns per block of an inner region
constexpr int KSTEP_B = NBLK * 16 * 2;  // 4096 B
constexpr int B_BLOCK = 4 * KSTEP_B;    // 16 KB: value j 0..15, value j 16..31, residue j 0..15, residue j 16..31
constexpr int KSTEP_BL = KMAX * 16 * 2; // 1024 B: leaf weights of one k-step (two features)
constexpr int LW_STAGE = 2 * KSTEP_BL;  // 2 KB: four features
constexpr int LW_RING = 4;
constexpr int SLOT_FLOATS = KMAX * TS;  // one a-stack slot: [32][128] floats
constexpr int LEAF_Q = 4;               // stages the input queue runs ahead
constexpr float kHalfRange = 240.f;     // |x'| below this: x'^2 < 65504
constexpr int TMEM_COLS = 512;

// barrier indices
constexpr int BAR_TILE = 9;             // per tile: opReady, accFull[2], accFree[2], leafFull[2], leafEmpty[2]
constexpr int BAR_OPREADY = 0, BAR_ACCFULL = 1, BAR_ACCFREE = 3, BAR_LEAFFULL = 5, BAR_LEAFEMPTY = 7;
constexpr int BAR_LEAFDONE = NTILE * BAR_TILE;         // [2]
constexpr int BAR_WFULL = BAR_LEAFDONE + NTILE;        // [4]
constexpr int BAR_WEMPTY = BAR_WFULL + 4;              // [4]
constexpr int BAR_LWFULL = BAR_WEMPTY + 4;             // [4]
constexpr int BAR_LWEMPTY = BAR_LWFULL + LW_RING;      // [4]
constexpr int BAR_DRAIN = BAR_LWEMPTY + LW_RING;
constexpr int NBARS = BAR_DRAIN + 1;

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
__device__ __forceinline__ void splitHalf(float v, float& hi, float& lo) {
  hi = __half2float(__float2half_rn(v));
  lo = v - hi;
}
__device__ __forceinline__ unsigned smemAddr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbarTry(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ void mbarArrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// contiguous global -> shared copy of `bytes` (a multiple of 16, both addresses 16-byte aligned); the barrier
// receives the byte count when the data has landed
__device__ __forceinline__ void bulkLoad(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
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
// The same load without the wait: the registers are written some time before the matching tmemWait32, which
// names them as in/out operands so that no use of them is scheduled ahead of it.
__device__ __forceinline__ void tmemLoad32Async(unsigned taddr, unsigned* r) {
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
}
__device__ __forceinline__ void tmemWait32(unsigned* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void fenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fenceAsyncProxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// two FP32 multiply-adds in one instruction: (acc.x, acc.y) += (a.x * b.x, a.y * b.y)
__device__ __forceinline__ void fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long pack2u(unsigned lo, unsigned hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ float sum2(unsigned long long v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}

// shared-memory matrix descriptor, K-major, no swizzle: start address, leading (K) byte offset, stride (M/N)
// byte offset, all in 16-byte units; descriptor version 1 (sm_100)
__device__ __forceinline__ unsigned long long smemDesc(unsigned addr, unsigned lboBytes, unsigned sboBytes) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lboBytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sboBytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

// Bounded wait shared by all roles: gives up after `limit` polls or as soon as another thread of the CTA has
// given up (the abort flag), and raises the flag itself in the first case.
struct Waiter {
  volatile int* abortFlag;
  unsigned limit;
  __device__ __forceinline__ bool wait(unsigned bar, unsigned parity) const {
    for (unsigned spin = 0; spin < limit; ++spin) {
      if (mbarTry(bar, parity)) return true;
      if ((spin & 63u) == 63u && *abortFlag) return false;
    }
    *abortFlag = 1;
    return false;
  }
};

// shared memory: [a-stack float x NTILE*aSlots*32*128][A operand 2 x 16 KB][weight ring ringBlocks x 16 KB]
//                [leaf weight ring 4 x 2 KB][barriers][tmem address][abort flag]
// Development aid: with PROFILE the first CTA's tile-0 lane 0, issuer and loader accumulate the cycles they
// spend per phase into prof[] (see layeredDualLaunch); the production instantiation carries none of it.
enum ProfSlot {
  P_W_TOTAL = 0, P_W_LEAF, P_W_LEAF_WAITEMPTY, P_W_LEAF_WAITDONE, P_W_INNER, P_W_INNER_PREP, P_W_INNER_WAITFULL,
  P_W_INNER_FOLD, P_W_DELIVER, P_W_FOLD_LDWAIT, P_W_LEAF_BUILD, P_W_LEAF_ARRIVE,
  P_I_TOTAL = 16, P_I_WAIT_WFULL, P_I_WAIT_OPREADY, P_I_WAIT_ACCFREE, P_I_WAIT_LWFULL, P_I_WAIT_LEAFFULL, P_I_LEAF, P_I_INNER, P_I_MMA, P_I_COMMIT, P_I_FENCE,
  P_L_TOTAL = 32, P_L_WAIT_WEMPTY,
  P_COUNT = 48
};
#define PROF_T() (PROFILE ? clock64() : 0ll)
#define PROF_ADD(slot, t0) do { if (PROFILE && profOn) prof[slot] += clock64() - (t0); } while (0)

template <bool MARGINAL, bool PROFILE>
__global__ void __launch_bounds__(NTHREADS, 1) layeredDualKernel(DualArgs a, const float* __restrict__ xt,
                                                                  float* __restrict__ out, unsigned long long n,
                                                                  int* __restrict__ status, long long* __restrict__ profOut) {
  long long prof[PROFILE ? P_COUNT : 1];
  if (PROFILE) for (int i = 0; i < P_COUNT; ++i) prof[i] = 0;
  const bool profOn = PROFILE && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x == 0 || threadIdx.x >= NWORK);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned warp = tid >> 5, lane = tid & 31;
  const int aSlots = a.aSlots, NB = a.ringBlocks;
  float* aStack = reinterpret_cast<float*>(smem_raw);
  unsigned char* abuf = smem_raw + (size_t)NTILE * aSlots * SLOT_FLOATS * 4;
  unsigned char* bring = abuf + NTILE * A_TILE;
  unsigned char* lwring = bring + (size_t)NB * B_BLOCK;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(lwring + LW_RING * LW_STAGE);
  unsigned* tmemSlot = reinterpret_cast<unsigned*>(bars + NBARS);
  volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
  const unsigned barBase = smemAddr(bars);
  auto bar = [&](int i) { return barBase + 8u * (unsigned)i; };
  const float NEG = __int_as_float(0xff800000);
  const Waiter w{abortFlag, a.spinLimit};

  if (tid == 0) {
    for (int t = 0; t < NTILE; ++t) {
      mbarInit(bar(t * BAR_TILE + BAR_OPREADY), 4);
      for (int b = 0; b < 2; ++b) {
        mbarInit(bar(t * BAR_TILE + BAR_ACCFULL + b), 1);
        mbarInit(bar(t * BAR_TILE + BAR_ACCFREE + b), 4);
        mbarInit(bar(t * BAR_TILE + BAR_LEAFFULL + b), 4);
        mbarInit(bar(t * BAR_TILE + BAR_LEAFEMPTY + b), 1);
      }
      mbarInit(bar(BAR_LEAFDONE + t), 1);
    }
    for (int i = BAR_WFULL; i < NBARS; ++i) mbarInit(bar(i), 1);
    *abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fenceBefore();
  __syncthreads();
  fenceAfter();
  const unsigned tmem = *tmemSlot;
  const unsigned long long npairs = (n + NTILE * TS - 1) / (NTILE * TS);
  bool failed = false;

  if (warp < 2 * 4) {
    // ================================ workers: one thread per sample ================================
    const unsigned t = warp >> 2;
    const unsigned r = tid & (TS - 1);
    const unsigned tmemAcc = tmem + t * 2 * NBLK + (((warp & 3u) * 32u) << 16);   // this warp's lane quarter
    float* myStack = aStack + (size_t)t * aSlots * SLOT_FLOATS + r;
    unsigned char* myA = abuf + t * A_TILE;
    const unsigned rowOff = (r >> 3) * 128 + (r & 7) * 16;   // this thread's row inside one k-half block
    const unsigned bT = t * BAR_TILE;
    unsigned phAccFull0 = 0, phAccFull1 = 0, phLeafEmpty0 = 0, phLeafEmpty1 = 0, phLeafDone = 0;
    unsigned pendEmpty0 = 0, pendEmpty1 = 0;

    const long long tW = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      const unsigned long long row = (pair * NTILE + t) * TS + r;
      const bool live = row < n;
      const float* __restrict__ xT = xt + (live ? row : 0);
      float xq[LEAF_Q][4];
      auto loadSlot = [&](int d, int g) {
        g = g < a.numLeafStages ? g : a.numLeafStages - 1;
#pragma unroll
        for (int u = 0; u < 4; ++u) xq[d][u] = xT[(size_t)__ldg(a.leafCols + g * 4 + u) * a.xtLd];
      };
      if (a.numLeafStages > 0) {
#pragma unroll
        for (int d = 0; d < LEAF_Q; ++d) loadSlot(d, d);
      } else {
#pragma unroll
        for (int d = 0; d < LEAF_Q; ++d)
#pragma unroll
          for (int u = 0; u < 4; ++u) xq[d][u] = 0.f;
      }
      float rootM = NEG, rootS = 0.f;
      float ea[KMAX];
      float ma = NEG, mb = NEG;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) ea[i] = 0.f;

      // a region's 32 outputs (base-2 logs) go where the program says
      auto deliver = [&](const DualStepDev& s, float* v) {
        if (s.dest == kDualDestStack) {
          float* dst = myStack + (size_t)s.destSlot * SLOT_FLOATS;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) dst[k * TS] = v[k];
        } else if (s.dest == kDualDestRegs) {
          ma = NEG;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) ma = fmaxf(ma, v[k]);
          const float za = ma == NEG ? 0.f : ma;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) ea[k] = ex2f(v[k] - za);
        } else if (s.dest == kDualDestOperand) {
          // right operand of the next step: 2^(v - max) as value / residue halves, straight into the MMA
          // operand buffer (k-steps 0, 1 = values of j 0..15, 16..31; k-steps 2, 3 = residues)
          mb = NEG;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) mb = fmaxf(mb, v[k]);
          const float zb = mb == NEG ? 0.f : mb;
          unsigned char* adst = myA + rowOff;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int kh = 0; kh < 2; ++kh) {
              float vh[8], vl[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) splitHalf(ex2f(v[16 * h + 8 * kh + q] - zb), vh[q], vl[q]);
              uint4 hi, lo;
              hi.x = packHalf2(vh[0], vh[1]); hi.y = packHalf2(vh[2], vh[3]);
              hi.z = packHalf2(vh[4], vh[5]); hi.w = packHalf2(vh[6], vh[7]);
              lo.x = packHalf2(vl[0], vl[1]); lo.y = packHalf2(vl[2], vl[3]);
              lo.z = packHalf2(vl[4], vl[5]); lo.w = packHalf2(vl[6], vl[7]);
              *reinterpret_cast<uint4*>(adst + h * KSTEP_A + kh * (KSTEP_A / 2)) = hi;
              *reinterpret_cast<uint4*>(adst + (2 + h) * KSTEP_A + kh * (KSTEP_A / 2)) = lo;
            }
          }
          fenceAsyncProxy();   // generic-proxy writes -> tensor core reads
        } else {
          // root part: fold its single output into the running log-sum
          const float x0 = v[0];
          if (x0 > rootM) { rootS = rootS * ex2f(rootM - x0) + 1.f; rootM = x0; }
          else if (x0 == x0 && x0 != NEG) rootS += ex2f(x0 - rootM);
          else if (x0 != x0) rootS = x0;
        }
      };

      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        float v[KMAX];
        if (s.op == kLeafRegion) {
          const long long tL = PROF_T();
          const int nst = s.numBlocks;
          bool redo = nst == 0;     // regions without tensor-core weights are computed by the FP32 loop below
          if (nst > 0) {
            const int nstPad = (nst + LEAF_Q - 1) / LEAF_Q * LEAF_Q;
#pragma unroll 1
            for (int st0 = 0; st0 < nstPad; st0 += LEAF_Q) {
#pragma unroll
              for (int d = 0; d < LEAF_Q; ++d) {
                const int st = st0 + d;
                if (st < nst && !failed) {
                  const int sb = d & 1;
                  // the MMAs that read this stage buffer two stages ago must be done
                  if (sb == 0 ? pendEmpty0 : pendEmpty1) {
                    const long long tq = PROF_T();
                    if (!w.wait(bar(bT + BAR_LEAFEMPTY + sb), sb == 0 ? phLeafEmpty0 : phLeafEmpty1)) failed = true;
                    PROF_ADD(P_W_LEAF_WAITEMPTY, tq);
                    if (sb == 0) { phLeafEmpty0 ^= 1; pendEmpty0 = 0; } else { phLeafEmpty1 ^= 1; pendEmpty1 = 0; }
                  }
                  if (!failed) {
                    const long long tb = PROF_T();
                    unsigned char* adst = myA + sb * LEAF_STAGE + rowOff;
                    const float* cen = a.leafCentres + (size_t)(s.stageBase + st) * 4;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                      const int f = st * 4 + u;
                      const float xv = xq[d][u];
                      const bool valid = f < s.numFeatures && (!MARGINAL || xv == xv);
                      const float xp = xv - __ldg(cen + u);
                      if (valid && !(fabsf(xp) < kHalfRange)) redo = true;
                      float xh, xl, sh, sl;
                      splitHalf(xp, xh, xl);
                      splitHalf(xp * xp, sh, sl);
                      uint4 q;
                      q.x = packHalf2(sh, sl);
                      q.y = packHalf2(sh, xh);
                      q.z = packHalf2(xl, xh);
                      q.w = 0x3C003C00u;   // (1, 1)
                      if (!valid) q = make_uint4(0u, 0u, 0u, 0u);
                      // feature 2 j of the stage is k 0..7 of k-step j, feature 2 j + 1 is k 8..15
                      *reinterpret_cast<uint4*>(adst + (u >> 1) * KSTEP_A + (u & 1) * (KSTEP_A / 2)) = q;
                    }
                    PROF_ADD(P_W_LEAF_BUILD, tb);
                    const long long ta = PROF_T();
                    fenceAsyncProxy();
                    __syncwarp();
                    if (lane == 0) mbarArrive(bar(bT + BAR_LEAFFULL + sb));
                    PROF_ADD(P_W_LEAF_ARRIVE, ta);
                    if (sb == 0) pendEmpty0 = 1; else pendEmpty1 = 1;
                  }
                }
                loadSlot(d, s.stageBase + st + LEAF_Q);
              }
            }
            // accumulator complete; the stage barriers' last completions are consumed as well, so that every
            // phase of every barrier is waited for exactly once
            const long long tq2 = PROF_T();
            if (!failed) { if (!w.wait(bar(BAR_LEAFDONE + t), phLeafDone)) failed = true; phLeafDone ^= 1; }
            PROF_ADD(P_W_LEAF_WAITDONE, tq2);
            if (!failed && pendEmpty0) { if (!w.wait(bar(bT + BAR_LEAFEMPTY), phLeafEmpty0)) failed = true; phLeafEmpty0 ^= 1; pendEmpty0 = 0; }
            if (!failed && pendEmpty1) { if (!w.wait(bar(bT + BAR_LEAFEMPTY + 1), phLeafEmpty1)) failed = true; phLeafEmpty1 ^= 1; pendEmpty1 = 0; }
            if (failed) break;
            fenceAfter();
            unsigned raw[KMAX];
            tmemLoad32(tmemAcc, raw);
            fenceBefore();   // the next MMA into this accumulator is ordered after these reads
#pragma unroll
            for (int k = 0; k < KMAX; ++k) v[k] = __uint_as_float(raw[k]);
          }
          if (redo) {
            // plain FP32 evaluation of this thread's row in the centred form (an input out of half-precision
            // range, or a region without tensor weights)
#pragma unroll
            for (int k = 0; k < KMAX; ++k) v[k] = 0.f;
            const float4* __restrict__ pbuf = a.leafParams + s.paramOffset;
            for (int f = 0; f < s.numFeatures; ++f) {
              const int col = __ldg(a.features + s.featOffset + f);
              float xv = xT[(size_t)col * a.xtLd];
              float m = 1.f;
              if (MARGINAL && xv != xv) { xv = 0.f; m = 0.f; }
              const float4* p = pbuf + (size_t)f * s.width;
#pragma unroll
              for (int k = 0; k < KMAX; ++k) {
                if (k < s.width) {
                  const float4 q = __ldg(p + k);
                  const float dx = xv - q.x;
                  const float tv = fmaf(dx * dx, q.y, q.z);
                  v[k] = MARGINAL ? fmaf(m, tv, v[k]) : v[k] + tv;
                }
              }
            }
          }
#pragma unroll
          for (int k = 0; k < KMAX; ++k)
            if (k >= s.width) v[k] = NEG;
          const long long tD = PROF_T();
          deliver(s, v);
          PROF_ADD(P_W_DELIVER, tD);
          PROF_ADD(P_W_LEAF, tL);
          continue;
        }
        // ---- inner region or root part -------------------------------------------------------------
        const long long tI = PROF_T();
        if (s.aSrc >= 0) {
          const float* src = myStack + (size_t)s.aSrc * SLOT_FLOATS;
          ma = NEG;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) { ea[k] = src[k * TS]; ma = fmaxf(ma, ea[k]); }
          const float za = ma == NEG ? 0.f : ma;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) ea[k] = ex2f(ea[k] - za);
        }
        const float base = ma + mb;
        // operand b is in the operand buffer (written and fenced by the previous step), both accumulators
        // have been read for the last time: the tensor core may start on this region
        fenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(bar(bT + BAR_OPREADY));
        unsigned long long ea2[KMAX / 2];
#pragma unroll
        for (int i = 0; i < KMAX / 2; ++i) ea2[i] = pack2(ea[2 * i], ea[2 * i + 1]);
        const float* scale = a.scales + s.scaleOffset;
        const int nblk = s.numBlocks;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) v[k] = NEG;
        PROF_ADD(P_W_INNER_PREP, tI);
#pragma unroll
        for (int nb = 0; nb < KMAX * KMAX / NBLK; ++nb) {
          if (nb < nblk && !failed) {
            const int b = nb & 1;
            float sc[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) sc[q] = __ldg(scale + 4 * nb + q);   // requested before the wait
            const long long tq = PROF_T();
            if (!w.wait(bar(bT + BAR_ACCFULL + b), b == 0 ? phAccFull0 : phAccFull1)) failed = true;
            PROF_ADD(P_W_INNER_WAITFULL, tq);
            if (b == 0) phAccFull0 ^= 1; else phAccFull1 ^= 1;
            const long long tf = PROF_T();
            if (!failed) {
              fenceAfter();
              // four sums per block; the accumulator columns of sum q + 1 travel from TMEM to registers while
              // sum q is folded (two register buffers)
              unsigned t0[KMAX], t1[KMAX];
              const unsigned tcol = tmemAcc + b * NBLK;
              const int nq = s.width - 4 * nb;   // sums of this block that exist (warp-uniform)
              auto dot = [&](const unsigned* tt, int q) {
                unsigned long long acc0 = 0ull, acc1 = 0ull, acc2 = 0ull, acc3 = 0ull;
#pragma unroll
                for (int i = 0; i < KMAX / 2; i += 4) {
                  fma2(acc0, ea2[i], pack2u(tt[2 * i], tt[2 * i + 1]));
                  fma2(acc1, ea2[i + 1], pack2u(tt[2 * i + 2], tt[2 * i + 3]));
                  fma2(acc2, ea2[i + 2], pack2u(tt[2 * i + 4], tt[2 * i + 5]));
                  fma2(acc3, ea2[i + 3], pack2u(tt[2 * i + 6], tt[2 * i + 7]));
                }
                v[4 * nb + q] = base + lg2f((sum2(acc0) + sum2(acc1)) + (sum2(acc2) + sum2(acc3))) + sc[q];
              };
              long long tw = PROF_T();
              tmemLoad32Async(tcol, t0);
              tmemWait32(t0);
              PROF_ADD(P_W_FOLD_LDWAIT, tw);
              if (nq > 1) tmemLoad32Async(tcol + KMAX, t1);
              dot(t0, 0);
              if (nq > 1) {
                tw = PROF_T();
                tmemWait32(t1);
                PROF_ADD(P_W_FOLD_LDWAIT, tw);
                if (nq > 2) tmemLoad32Async(tcol + 2 * KMAX, t0);
                dot(t1, 1);
              }
              if (nq > 2) {
                tw = PROF_T();
                tmemWait32(t0);
                PROF_ADD(P_W_FOLD_LDWAIT, tw);
                if (nq > 3) tmemLoad32Async(tcol + 3 * KMAX, t1);
                dot(t0, 2);
              }
              if (nq > 3) {
                tw = PROF_T();
                tmemWait32(t1);
                PROF_ADD(P_W_FOLD_LDWAIT, tw);
                dot(t1, 3);
              }
              // a later block's MMAs overwrite this accumulator: order the reads before the arrival that
              // allows them (the last two blocks are covered by the next region's operand arrival)
              fenceBefore();
              if (nb + 2 < nblk) {
                __syncwarp();
                if (lane == 0) mbarArrive(bar(bT + BAR_ACCFREE + b));
              }
            }
            PROF_ADD(P_W_INNER_FOLD, tf);
          }
        }
        if (failed) break;
        const long long tD = PROF_T();
        deliver(s, v);
        PROF_ADD(P_W_DELIVER, tD);
        PROF_ADD(P_W_INNER, tI);
      }
      if (live && !failed) out[row] = (rootM + lg2f(rootS)) * 0x1.62e43p-1f;
    }
    PROF_ADD(P_W_TOTAL, tW);
  } else if (warp == 8) {
    // ================================ MMA issuer ====================================================
    const unsigned idescLeaf = (1u << 4) | ((unsigned)(KMAX >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
    const unsigned idescSum = (1u << 4) | ((unsigned)(NBLK >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
    // Descriptors of the operand areas' first blocks, built once: a block further on adds its byte offset / 16
    // to the start-address field (the sum stays inside the field: shared memory ends below 256 KB).  Building a
    // descriptor from scratch costs a dozen dependent integer instructions; with one thread issuing every MMA
    // of the CTA that latency would sit in front of each of them.
    const unsigned long long aDesc[NTILE] = {smemDesc(smemAddr(abuf), KSTEP_A / 2, 128),
                                             smemDesc(smemAddr(abuf) + A_TILE, KSTEP_A / 2, 128)};
    const unsigned long long bDesc0 = smemDesc(smemAddr(bring), KSTEP_B / 2, 128);
    const unsigned long long lwDesc0 = smemDesc(smemAddr(lwring), KSTEP_BL / 2, 128);
    unsigned phOpReady0 = 0, phOpReady1 = 0, phAccFree00 = 0, phAccFree01 = 0, phAccFree10 = 0, phAccFree11 = 0;
    unsigned phLeafFull00 = 0, phLeafFull01 = 0, phLeafFull10 = 0, phLeafFull11 = 0;
    unsigned wCount = 0, lwCount = 0;   // blocks / leaf stages consumed so far: ring slot and parity
    bool withheld = a.testWithholdCommit == 0;
    const long long tIs = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        const long long tStep = PROF_T();
        if (s.op == kLeafRegion) {
          const int nst = s.numBlocks;
#pragma unroll 1
          for (int st = 0; st < nst && !failed; ++st) {
            const unsigned ring = lwCount % LW_RING;
            const long long tq = PROF_T();
            if (!w.wait(bar(BAR_LWFULL + ring), (lwCount / LW_RING) & 1)) { failed = true; break; }
            PROF_ADD(P_I_WAIT_LWFULL, tq);
            const int sb = st & 1;
            const unsigned long long lwd = lwDesc0 + (unsigned)((ring * LW_STAGE) >> 4);
#pragma unroll
            for (int t = 0; t < NTILE; ++t) {
              if (failed) break;
              const long long tq3 = PROF_T();
              unsigned& ph = t == 0 ? (sb == 0 ? phLeafFull00 : phLeafFull01) : (sb == 0 ? phLeafFull10 : phLeafFull11);
              if (!w.wait(bar(t * BAR_TILE + BAR_LEAFFULL + sb), ph)) { failed = true; break; }
              PROF_ADD(P_I_WAIT_LEAFFULL, tq3);
              ph ^= 1;
              if (lane == 0) {
                fenceAfter();
                const unsigned long long ad = aDesc[t] + (unsigned)((sb * LEAF_STAGE) >> 4);
                mmaF16(tmem + t * 2 * NBLK, ad, lwd, idescLeaf, st ? 1u : 0u);
                mmaF16(tmem + t * 2 * NBLK, ad + (KSTEP_A >> 4), lwd + (KSTEP_BL >> 4), idescLeaf, 1u);
                mmaCommit(bar(t * BAR_TILE + BAR_LEAFEMPTY + sb));
                if (st == nst - 1) mmaCommit(bar(BAR_LEAFDONE + t));
              }
              __syncwarp();
            }
            if (lane == 0 && !failed) mmaCommit(bar(BAR_LWEMPTY + ring));
            __syncwarp();
            ++lwCount;
          }
          PROF_ADD(P_I_LEAF, tStep);
          continue;
        }
        const int nblk = s.numBlocks;
#pragma unroll 1
        for (int nb = 0; nb < nblk && !failed; ++nb) {
          const unsigned ring = wCount % (unsigned)NB;
          const long long tq = PROF_T();
          if (!w.wait(bar(BAR_WFULL + ring), (wCount / (unsigned)NB) & 1)) { failed = true; break; }
          PROF_ADD(P_I_WAIT_WFULL, tq);
          const int b = nb & 1;
          const unsigned long long bdBlock = bDesc0 + (unsigned)((ring * B_BLOCK) >> 4);
#pragma unroll
          for (int t = 0; t < NTILE; ++t) {
            if (failed) break;
            if (nb == 0) {
              const long long tq4 = PROF_T();
              unsigned& ph = t == 0 ? phOpReady0 : phOpReady1;
              if (!w.wait(bar(t * BAR_TILE + BAR_OPREADY), ph)) { failed = true; break; }
              PROF_ADD(P_I_WAIT_OPREADY, tq4);
              ph ^= 1;
            } else if (nb >= 2) {
              const long long tq5 = PROF_T();
              unsigned& ph = t == 0 ? (b == 0 ? phAccFree00 : phAccFree01) : (b == 0 ? phAccFree10 : phAccFree11);
              if (!w.wait(bar(t * BAR_TILE + BAR_ACCFREE + b), ph)) { failed = true; break; }
              PROF_ADD(P_I_WAIT_ACCFREE, tq5);
              ph ^= 1;
            }
            if (lane == 0) {
              const long long tfz = PROF_T();
              fenceAfter();
              PROF_ADD(P_I_FENCE, tfz);
              const long long tmm = PROF_T();
              const unsigned d = tmem + t * 2 * NBLK + b * NBLK;
              // value x value, residue x value, value x residue, each over j 0..15 and j 16..31
#pragma unroll
              for (int m = 0; m < 6; ++m) {
                const int aks = (m < 4) ? m : m - 4;   // A k-step: 0,1 value; 2,3 residue; 0,1 value
                const int bks = (m < 2) ? m : m - 2;   // B k-step: 0,1 value; 0,1 value; 2,3 residue
                mmaF16(d, aDesc[t] + (unsigned)((aks * KSTEP_A) >> 4), bdBlock + (unsigned)((bks * KSTEP_B) >> 4), idescSum, m ? 1u : 0u);
              }
              PROF_ADD(P_I_MMA, tmm);
              const long long tcm = PROF_T();
              // self-test: leave out one commit, so that the workers' wait for it runs out
              if (!withheld) withheld = true;
              else mmaCommit(bar(t * BAR_TILE + BAR_ACCFULL + b));
              PROF_ADD(P_I_COMMIT, tcm);
            }
            __syncwarp();
          }
          if (lane == 0 && !failed) mmaCommit(bar(BAR_WEMPTY + ring));
          __syncwarp();
          ++wCount;
        }
        PROF_ADD(P_I_INNER, tStep);
      }
    }
    PROF_ADD(P_I_TOTAL, tIs);
    // every MMA issued by this warp has completed when this barrier flips (also after a failure)
    if (lane == 0) mmaCommit(bar(BAR_DRAIN));
    __syncwarp();
    w.wait(bar(BAR_DRAIN), 0);
  } else if (warp == 9) {
    // ================================ inner-region weight loader =====================================
    unsigned issued = 0;
    const unsigned bAddr = smemAddr(bring);
    const long long tLs = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        if (s.op == kLeafRegion) continue;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(a.frags) + s.fragOffset;
        for (int nb = 0; nb < s.numBlocks && !failed; ++nb) {
          const unsigned ring = issued % (unsigned)NB;
          // the slot's previous block has been multiplied for both tiles
          const long long tq = PROF_T();
          if (issued >= (unsigned)NB && !w.wait(bar(BAR_WEMPTY + ring), ((issued / (unsigned)NB) - 1) & 1)) { failed = true; break; }
          PROF_ADD(P_L_WAIT_WEMPTY, tq);
          if (lane == 0) {
            mbarExpectTx(bar(BAR_WFULL + ring), B_BLOCK);
            bulkLoad(bAddr + ring * B_BLOCK, src + (size_t)nb * B_BLOCK, B_BLOCK, bar(BAR_WFULL + ring));
          }
          __syncwarp();
          ++issued;
        }
      }
    }
    PROF_ADD(P_L_TOTAL, tLs);
    // copies still in flight must land before the CTA's shared memory goes away
    const unsigned pending = issued < (unsigned)NB ? issued : (unsigned)NB;
    for (unsigned i = issued - pending; i < issued; ++i) w.wait(bar(BAR_WFULL + i % (unsigned)NB), (i / (unsigned)NB) & 1);
  } else {
    // ================================ leaf weight loader ============================================
    unsigned issued = 0;
    const unsigned lwAddr = smemAddr(lwring);
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        if (s.op != kLeafRegion) continue;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(a.frags) + s.fragOffset;
        for (int st = 0; st < s.numBlocks && !failed; ++st) {
          const unsigned ring = issued % LW_RING;
          if (issued >= LW_RING && !w.wait(bar(BAR_LWEMPTY + ring), ((issued / LW_RING) - 1) & 1)) { failed = true; break; }
          if (lane == 0) {
            mbarExpectTx(bar(BAR_LWFULL + ring), LW_STAGE);
            bulkLoad(lwAddr + ring * LW_STAGE, src + (size_t)st * LW_STAGE, LW_STAGE, bar(BAR_LWFULL + ring));
          }
          __syncwarp();
          ++issued;
        }
      }
    }
    const unsigned pending = issued < LW_RING ? issued : LW_RING;
    for (unsigned i = issued - pending; i < issued; ++i) w.wait(bar(BAR_LWFULL + i % LW_RING), (i / LW_RING) & 1);
  }

  // ---- common exit: report, wait for the other roles' drains, free the tensor memory --------------------
  if (failed || *abortFlag) atomicExch(status, 1);
  if (PROFILE && profOn) {
    const int lo = tid == 0 ? 0 : (warp == 8 ? 16 : (warp == 9 ? 32 : 40)), hi = tid == 0 ? 16 : (warp == 8 ? 32 : (warp == 9 ? 40 : 48));
    for (int i = lo; i < hi; ++i) profOut[i] = prof[i];
  }
  fenceBefore();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

size_t layeredDualSmemBytes(int aSlots, int ringBlocks) {
  return (size_t)NTILE * aSlots * SLOT_FLOATS * 4 + NTILE * A_TILE + (size_t)ringBlocks * B_BLOCK + LW_RING * LW_STAGE +
         NBARS * 8 + 16;
}

int layeredDualThreads() { return NTHREADS; }

cudaError_t layeredDualLaunch(const DualArgs& a, const float* xt, float* out, size_t n, int grid, size_t smem, int* status,
                              cudaStream_t stream) {
  auto run = [&](auto kernel, long long* prof) -> cudaError_t {
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(kernel), smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, NTHREADS, smem, stream>>>(a, xt, out, (unsigned long long)n, status, prof);
    return cudaGetLastError();
  };
  if (std::getenv("SPNB_DUAL_PROFILE")) {
    // development aid: per-phase cycle counts of the first CTA, printed after the launch (synchronous)
    long long* dProf = nullptr;
    if (cudaMalloc(&dProf, P_COUNT * sizeof(long long)) != cudaSuccess) return cudaErrorMemoryAllocation;
    cudaMemset(dProf, 0, P_COUNT * sizeof(long long));
    cudaError_t e = a.marginal ? run(layeredDualKernel<true, true>, dProf) : run(layeredDualKernel<false, true>, dProf);
    long long h[P_COUNT];
    cudaMemcpy(h, dProf, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(dProf);
    static const char* names[P_COUNT] = {"w_total", "w_leaf", "w_leaf_wait_empty", "w_leaf_wait_done", "w_inner", "w_inner_prep",
        "w_inner_wait_full", "w_inner_fold", "w_deliver", "w_fold_ldwait", "w_leaf_build", "w_leaf_arrive", 0, 0, 0, 0,
        "i_total", "i_wait_wfull", "i_wait_opready", "i_wait_accfree", "i_wait_lwfull", "i_wait_leaffull", "i_leaf", "i_inner", "i_mma", "i_commit", "i_fence", 0, 0, 0, 0, 0,
        "l_total", "l_wait_wempty"};
    std::fprintf(stderr, "[dual profile] n=%zu grid=%d:", n, grid);
    for (int i = 0; i < P_COUNT; ++i) if (names[i]) std::fprintf(stderr, " %s=%lld", names[i], h[i]);
    std::fprintf(stderr, "\n");
    return e;
  }
  return a.marginal ? run(layeredDualKernel<true, false>, nullptr) : run(layeredDualKernel<false, false>, nullptr);
}

}  // namespace spnb
