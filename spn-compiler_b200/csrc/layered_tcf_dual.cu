// Layered (RAT-SPN-style) SPN evaluation on the 5th-generation tensor cores, two sample tiles per CTA.
//
// Same arithmetic as layered_tcf.cu (factorised inner regions T = eb x W on tcgen05.mma with TMEM accumulators,
// S_k = sum_i ea_i T[(k,i)] on the CUDA cores; leaf regions as [x'^2, x', 1] x parameters, all operands half
// precision carried as value + rounding residue), but scheduled so that the tensor pipe does not wait for
// one tile's dependency chain:
//
//   * A CTA owns TWO tiles of 128 samples.  Both walk the same region program, so every block of weights that
//     is brought into shared memory is used by two groups of MMAs (half the L2 -> shared traffic per sample),
//     and while the threads of one tile fold an accumulator the tensor core works for the other.
//   * Warp roles: warps 0-3 = tile 0, warps 4-7 = tile 1 (thread = sample = TMEM lane); warps 8 and 9 issue
//     the MMAs of tile 0 and tile 1; warp 10 streams inner-region weights, warp 11 everything a leaf stage
//     needs (its weights, the eight features' inputs for the 256 samples of the tile pair out of the
//     feature-major copy, the eight centres) with bulk asynchronous copies (cp.async.bulk global -> shared,
//     completion counted on an mbarrier, this CTA only).  No worker thread loads inputs from global memory.
//     Roles meet only through mbarriers; there is no CTA-wide barrier inside the tile loop.
//   * A region's 32 outputs travel as a block normalised to a maximum of 1 plus one base-2 log scale per
//     sample, which is what the consumer's contraction needs: inner regions take one logarithm per sample
//     instead of 32 logarithms and 64 exponentials.  In the post-order walk the right operand (b) of a region
//     is always produced by the step directly before it: its producer writes it straight into the tile's MMA
//     operand buffer (value / residue halves).  Left operands (a) wait in a small "a-stack" (one 16.5 KB slot
//     per pending left operand; the outermost slot, written and read once per repetition, lives in global
//     memory), or stay in registers when the right sibling is a single leaf region.
//   * Leaf stages (eight features, K = 64) never touch shared memory on the operand side: a thread builds its
//     sample's 64 half-precision entries in registers and stores them with tcgen05.st into tensor-memory
//     columns of its tile's second accumulator (idle while a leaf region runs); the MMAs read their left
//     operand from there.
//   * TMEM: 512 columns = 2 tiles x 2 accumulators x 128 columns; a leaf region accumulates in the first 32
//     columns of its tile's accumulator 0.
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
constexpr int NTHREADS = NWORK + 128;   // + one MMA issuer warp per tile, weight loader warp, leaf loader warp
constexpr int KSTEP_A = TS * 16 * 2;    // 4096 B: one 128 x 16 operand block [k-half 2][row group 16][row 8][8 halves]
constexpr int A_TILE = 4 * KSTEP_A;     // 16 KB per tile: the inner regions' right operand (4 k-steps)
constexpr int STAGE_FEATS = 8;          // features per leaf stage: K = 64, four MMAs
constexpr int STAGE_COLS = 4 * STAGE_FEATS;   // TMEM columns of one stage's operand rows (eight halves per feature)
constexpr int NBLK = 128;               // (k,i) columns per block of an inner region
constexpr int KSTEP_B = NBLK * 16 * 2;  // 4096 B
constexpr int B_BLOCK = 4 * KSTEP_B;    // 16 KB: value j 0..15, value j 16..31, residue j 0..15, residue j 16..31
constexpr int KSTEP_BL = KMAX * 16 * 2; // 1024 B: leaf weights of one k-step (two features)
constexpr int LW_STAGE = 4 * KSTEP_BL;  // 4 KB: eight features
constexpr int W_RING_MAX = 6;            // weight blocks in flight, at most
constexpr int LW_RING_MAX = 7;           // leaf stages in flight, at most (tensor-memory columns for their operand rows)
// one leaf ring slot: the stage's weights, its eight features' inputs for the 256 samples of the tile pair,
// its eight centres (padded to 128 bytes)
constexpr int LEAF_X = STAGE_FEATS * NTILE * TS * 4;
constexpr int LEAF_SLOT_TX = LW_STAGE + LEAF_X + STAGE_FEATS * 4;
constexpr int LEAF_SLOT = LW_STAGE + LEAF_X + 128;
constexpr int SLOT_FLOATS = (KMAX + 1) * TS;  // one a-stack slot: [32][128] normalised values, then [128] log2 scales
// Tensor-memory columns (relative to the tile's first accumulator) of the operand rows of the leaf stage in ring
// slot `slot`: slots 0-3 fill the second accumulator, slots 4-6 the columns of the first accumulator behind the
// 32 a leaf region accumulates into.  No inner region is in flight on the tile while a leaf region runs.
__device__ __forceinline__ unsigned leafOperandCol(unsigned slot) {
  return slot < 4u ? (unsigned)NBLK + slot * STAGE_COLS : (slot - 3u) * STAGE_COLS;
}
constexpr float kHalfRange = 240.f;     // |x'| below this: x'^2 < 65504
constexpr int TMEM_COLS = 512;

// barrier indices
constexpr int BAR_TILE = 5 + LW_RING_MAX; // per tile: opReady, accFull[2], accFree[2], leafFull[LW_RING_MAX]
constexpr int BAR_OPREADY = 0, BAR_ACCFULL = 1, BAR_ACCFREE = 3, BAR_LEAFFULL = 5;
constexpr int BAR_LEAFDONE = NTILE * BAR_TILE;         // [2]
constexpr int BAR_WFULL = BAR_LEAFDONE + NTILE;        // [W_RING_MAX] weight block landed
constexpr int BAR_WEMPTY = BAR_WFULL + W_RING_MAX;     // [W_RING_MAX] both tiles' MMAs on the block done (two commits)
constexpr int BAR_LWFULL = BAR_WEMPTY + W_RING_MAX;    // [LW_RING_MAX] leaf stage (weights, inputs, centres) landed
constexpr int BAR_LWEMPTY = BAR_LWFULL + LW_RING_MAX;  // [LW_RING_MAX] both tiles' MMAs on the stage done (two commits)
constexpr int BAR_DRAIN = BAR_LWEMPTY + LW_RING_MAX;   // [2] per issuer
constexpr int NBARS = BAR_DRAIN + NTILE;

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
// v = hi + lo with hi exactly representable in half precision (for |v| in the normal half range): hi keeps the
// top 11 significant bits of v (truncation: one integer instruction instead of two format conversions, which
// run at a quarter of the FP32 rate), lo = v - hi is exact in FP32 and is rounded to half when it is packed.
__device__ __forceinline__ void splitHalf(float v, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
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
// this thread's 32 consecutive columns (lane = its sample) from registers to TMEM
__device__ __forceinline__ void tmemStore32(unsigned taddr, const unsigned* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// MMA whose left operand is read from tensor memory (lane = row, two half-precision K elements per column)
__device__ __forceinline__ void mmaF16TmemA(unsigned d, unsigned a, unsigned long long bd, unsigned idesc,
                                            unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d),
      "r"(a), "l"(bd), "r"(idesc), "r"(accumulate)
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
// Development aid: with PROFILE the first CTA's tile-0 lane 0, issuer 0 and the loaders accumulate the cycles
// they spend per phase into prof[] (see layeredDualLaunch); the production instantiation carries none of it.
enum ProfSlot {
  P_W_TOTAL = 0, P_W_LEAF, P_W_LEAF_WAITDATA, P_W_LEAF_WAITEMPTY, P_W_LEAF_WAITDONE, P_W_INNER, P_W_INNER_PREP,
  P_W_INNER_WAITFULL, P_W_INNER_FOLD, P_W_DELIVER, P_W_LEAF_FENCE, P_W_LEAF_BUILD,
  P_I_TOTAL = 16, P_I_WAIT_OPREADY, P_I_WAIT_ACCFREE, P_I_WAIT_WFULL, P_I_WAIT_LEAFFULL, P_I_LEAF, P_I_INNER,
  P_L_TOTAL = 32, P_L_WAIT,
  P_LL_TOTAL = 40, P_LL_WAIT,
  P_COUNT = 48
};
#define PROF_T() (PROFILE ? clock64() : 0ll)
#define PROF_ADD(slot, t0) do { if (PROFILE && profOn) prof[slot] += clock64() - (t0); } while (0)

// shared memory: [a-stack float x NTILE*aSlots*32*128][A operand 2 x 16 KB][weight ring ringBlocks x 16 KB]
//                [leaf ring 4 x (weights 2 KB, inputs 4 features x 256 samples, 4 centres)][barriers]
//                [tmem address][abort flag]
template <bool MARGINAL, bool PACKED, bool PROFILE>
__global__ void __launch_bounds__(NTHREADS, 1) layeredDualKernel(DualArgs a, const float* __restrict__ xt,
                                                                  float* __restrict__ out, unsigned long long n,
                                                                  int* __restrict__ status, long long* __restrict__ profOut) {
  long long prof[PROFILE ? P_COUNT : 1];
  if (PROFILE) for (int i = 0; i < P_COUNT; ++i) prof[i] = 0;
  const bool profOn = PROFILE && blockIdx.x == 0 && (threadIdx.x & 31) == 0 &&
                      (threadIdx.x == 0 || threadIdx.x == NWORK || threadIdx.x >= NWORK + 64);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned warp = tid >> 5, lane = tid & 31;
  const int aSlots = a.aSlots, NB = a.ringBlocks, LR = a.leafRing;
  float* aStack = reinterpret_cast<float*>(smem_raw);
  unsigned char* abuf = smem_raw + (size_t)NTILE * aSlots * SLOT_FLOATS * 4;
  unsigned char* bring = abuf + NTILE * A_TILE;
  unsigned char* lring = bring + (size_t)NB * B_BLOCK;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(lring + (size_t)LR * LEAF_SLOT);
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
      }
      for (int i = 0; i < LW_RING_MAX; ++i) mbarInit(bar(t * BAR_TILE + BAR_LEAFFULL + i), 4);
      mbarInit(bar(BAR_LEAFDONE + t), 1);
      mbarInit(bar(BAR_DRAIN + t), 1);
    }
    for (int i = 0; i < W_RING_MAX; ++i) {
      mbarInit(bar(BAR_WFULL + i), 1);
      mbarInit(bar(BAR_WEMPTY + i), NTILE);
    }
    for (int i = 0; i < LW_RING_MAX; ++i) {
      mbarInit(bar(BAR_LWFULL + i), 1);
      mbarInit(bar(BAR_LWEMPTY + i), NTILE);
    }
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
    // a-stack slot s lives in shared memory at index s - gSlots; the gSlots outermost (longest-lived) slots live
    // in a per-CTA area of global memory instead, written once and read once per repetition
    const int gSlots = a.globalSlots;
    float* myStack = aStack + (size_t)t * aSlots * SLOT_FLOATS + r;
    float* myGlobal = a.globalStack + ((size_t)blockIdx.x * NTILE + t) * (size_t)(gSlots > 0 ? gSlots : 1) * SLOT_FLOATS + r;
    auto slotPtr = [&](int slot) -> float* {
      return slot < gSlots ? myGlobal + (size_t)slot * SLOT_FLOATS : myStack + (size_t)(slot - gSlots) * SLOT_FLOATS;
    };
    unsigned char* myA = abuf + t * A_TILE;
    const unsigned rowOff = (r >> 3) * 128 + (r & 7) * 16;   // this thread's row inside one k-half block
    const unsigned bT = t * BAR_TILE;
    unsigned phAccFull0 = 0, phAccFull1 = 0, phLeafDone = 0;
    unsigned leafSeen = 0, leafRing = 0, leafPar = 0;   // leaf stages consumed so far; ring slot and parity of the next

    const long long tW = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      const unsigned long long row = (pair * NTILE + t) * TS + r;
      const bool live = row < n;
      const float* __restrict__ xT = xt + (live ? row : 0);
      float rootM = NEG, rootS = 0.f;
      float ea[KMAX];
      float ma = NEG, mb = NEG;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) ea[i] = 0.f;

      // A region's outputs travel as a block of 32 values normalised to a maximum of 1 plus one base-2 log scale
      // per sample (value_k = scale + log2(lin_k)): exactly what the consumer's contraction needs, so inner
      // regions never take per-value logarithms or exponentials.  The block goes where the program says.
      auto deliver = [&](const DualStepDev& s, const float* lin, float scale) {
        if (s.dest == kDualDestStack) {
          float* dst = slotPtr(s.destSlot);
#pragma unroll
          for (int k = 0; k < KMAX; ++k) dst[k * TS] = lin[k];
          dst[KMAX * TS] = scale;
        } else if (s.dest == kDualDestRegs) {
#pragma unroll
          for (int k = 0; k < KMAX; ++k) ea[k] = lin[k];
          ma = scale;
        } else if (s.dest == kDualDestOperand) {
          // right operand of the next step: value / residue halves straight into the MMA operand buffer
          // (k-steps 0, 1 = values of j 0..15, 16..31; k-steps 2, 3 = residues)
          mb = scale;
          unsigned char* adst = myA + rowOff;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int kh = 0; kh < 2; ++kh) {
              float vh[8], vl[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) splitHalf(lin[16 * h + 8 * kh + q], vh[q], vl[q]);
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
          const float x0 = scale + lg2f(lin[0]);
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
#pragma unroll 1
            for (int st = 0; st < nst && !failed; ++st) {
              // The stage's inputs and centres have landed in the leaf ring (its weights with them).  The loader
              // refilled the slot only after both tiles' MMAs on the slot's previous stage had completed, so
              // this tile's operand buffer of the same index in tensor memory is free as well.
              {
                const long long tq = PROF_T();
                if (!w.wait(bar(BAR_LWFULL + (int)leafRing), leafPar)) { failed = true; break; }
                PROF_ADD(P_W_LEAF_WAITDATA, tq);
              }
              const long long tb = PROF_T();
              const unsigned char* slot = lring + leafRing * LEAF_SLOT;
              const float* xin = reinterpret_cast<const float*>(slot + LW_STAGE) + t * TS + r;   // [feature][256 samples]
              const float* cen = reinterpret_cast<const float*>(slot + LW_STAGE + LEAF_X);
              unsigned rowsA[STAGE_COLS];
#pragma unroll
              for (int u = 0; u < STAGE_FEATS; ++u) {
                const int f = st * STAGE_FEATS + u;
                const float xv = xin[u * NTILE * TS];
                const bool valid = f < s.numFeatures && (!MARGINAL || xv == xv);
                const float xp = xv - cen[u];
                if (valid && !(fabsf(xp) < kHalfRange)) redo = true;
                float xh, xl, sh, sl;
                splitHalf(xp, xh, xl);
                splitHalf(xp * xp, sh, sl);
                // eight K entries of the feature: (sh, sl, sh, xh, xl, xh, 1, 1); a missing input contributes zeros
                rowsA[4 * u] = valid ? packHalf2(sh, sl) : 0u;
                rowsA[4 * u + 1] = valid ? packHalf2(sh, xh) : 0u;
                rowsA[4 * u + 2] = valid ? packHalf2(xl, xh) : 0u;
                rowsA[4 * u + 3] = valid ? 0x3C003C00u : 0u;
              }
              // operand rows of this stage: tensor-memory columns of the tile's second accumulator, which no
              // inner region uses while a leaf region runs (feature 2 j, 2 j + 1 = the 16 K entries of MMA j)
              tmemStore32(tmemAcc + leafOperandCol(leafRing), rowsA);
              PROF_ADD(P_W_LEAF_BUILD, tb);
              fenceBefore();
              __syncwarp();
              if (lane == 0) mbarArrive(bar(bT + BAR_LEAFFULL + (int)leafRing));
              ++leafSeen;
              if (++leafRing == (unsigned)LR) { leafRing = 0; leafPar ^= 1; }
            }
            // accumulator complete
            const long long tq2 = PROF_T();
            if (!failed) { if (!w.wait(bar(BAR_LEAFDONE + t), phLeafDone)) failed = true; phLeafDone ^= 1; }
            PROF_ADD(P_W_LEAF_WAITDONE, tq2);
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
          const long long tD = PROF_T();
          {
            // base-2 log densities -> normalised block: the only place a region takes 32 exponentials
            float mx = NEG;
#pragma unroll
            for (int k = 0; k < KMAX; ++k) {
              if (k >= s.width) v[k] = NEG;
              mx = fmaxf(mx, v[k]);
            }
            const float z = mx == NEG ? 0.f : mx;
#pragma unroll
            for (int k = 0; k < KMAX; ++k) v[k] = ex2f(v[k] - z);
            deliver(s, v, mx);
          }
          PROF_ADD(P_W_DELIVER, tD);
          PROF_ADD(P_W_LEAF, tL);
          continue;
        }
        // ---- inner region or root part -------------------------------------------------------------
        const long long tI = PROF_T();
        if (s.aSrc >= 0) {
          const float* src = slotPtr(s.aSrc);
#pragma unroll
          for (int k = 0; k < KMAX; ++k) ea[k] = src[k * TS];
          ma = src[KMAX * TS];
        }
        const float base = ma + mb;
        // operand b is in the operand buffer (written and fenced by the previous step), both accumulators
        // have been read for the last time: the tensor core may start on this region
        fenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(bar(bT + BAR_OPREADY));
        unsigned long long ea2[PACKED ? KMAX / 2 : 1];
        if (PACKED) {
#pragma unroll
          for (int i = 0; i < KMAX / 2; ++i) ea2[i] = pack2(ea[2 * i], ea[2 * i + 1]);
        }
        const float* scale = a.scaleMul + s.scaleOffset;
        const int nblk = s.numBlocks;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) v[k] = 0.f;
        PROF_ADD(P_W_INNER_PREP, tI);
#pragma unroll
        for (int nb = 0; nb < KMAX * KMAX / NBLK; ++nb) {
          if (nb < nblk && !failed) {
            const int b = nb & 1;
            const long long tq = PROF_T();
            if (!w.wait(bar(bT + BAR_ACCFULL + b), b == 0 ? phAccFull0 : phAccFull1)) failed = true;
            PROF_ADD(P_W_INNER_WAITFULL, tq);
            if (b == 0) phAccFull0 ^= 1; else phAccFull1 ^= 1;

            const long long tf = PROF_T();
            if (!failed) {
              fenceAfter();
              // four sums per block; the accumulator columns of sum q + 1 travel from TMEM to registers while
              // sum q is folded (two register buffers).  (Requesting the next block's first columns into the free
              // buffer under the last fold of this block keeps 32 more registers alive at the 168-register cap:
              // 468 bytes of spills instead of 136, 210 ms against 188 ms for 2 M samples.)
              unsigned t0[KMAX], t1[KMAX];
              const unsigned tcol = tmemAcc + b * NBLK;
              const int nq = s.width - 4 * nb;   // sums of this block that exist (warp-uniform)
              auto dot = [&](const unsigned* tt, int q) {
                float total;
                if (PACKED) {
                  unsigned long long acc0 = 0ull, acc1 = 0ull, acc2 = 0ull, acc3 = 0ull;
#pragma unroll
                  for (int i = 0; i < KMAX / 2; i += 4) {
                    fma2(acc0, ea2[i], pack2u(tt[2 * i], tt[2 * i + 1]));
                    fma2(acc1, ea2[i + 1], pack2u(tt[2 * i + 2], tt[2 * i + 3]));
                    fma2(acc2, ea2[i + 2], pack2u(tt[2 * i + 4], tt[2 * i + 5]));
                    fma2(acc3, ea2[i + 3], pack2u(tt[2 * i + 6], tt[2 * i + 7]));
                  }
                  total = (sum2(acc0) + sum2(acc1)) + (sum2(acc2) + sum2(acc3));
                } else {
                  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
                  for (int i = 0; i < KMAX; i += 4) {
                    acc0 = fmaf(ea[i], __uint_as_float(tt[i]), acc0);
                    acc1 = fmaf(ea[i + 1], __uint_as_float(tt[i + 1]), acc1);
                    acc2 = fmaf(ea[i + 2], __uint_as_float(tt[i + 2]), acc2);
                    acc3 = fmaf(ea[i + 3], __uint_as_float(tt[i + 3]), acc3);
                  }
                  total = (acc0 + acc1) + (acc2 + acc3);
                }
                v[4 * nb + q] = total;   // the logarithms of all sums are taken together after the last block
              };
              tmemLoad32Async(tcol, t0);
              tmemWait32(t0);
              if (nq > 1) tmemLoad32Async(tcol + KMAX, t1);
              dot(t0, 0);
              if (nq > 1) {
                tmemWait32(t1);
                if (nq > 2) tmemLoad32Async(tcol + 2 * KMAX, t0);
                dot(t1, 1);
              }
              if (nq > 2) {
                tmemWait32(t0);
                if (nq > 3) tmemLoad32Async(tcol + 3 * KMAX, t1);
                dot(t0, 2);
              }
              if (nq > 3) {
                tmemWait32(t1);
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
        {
          // sums -> normalised block: the sums were contracted with each weight row divided by its largest
          // weight; multiply that back in, divide by the largest sum and keep its logarithm as the scale
          float mx = 0.f;
#pragma unroll
          for (int k = 0; k < KMAX; ++k) {
            v[k] = k < s.width ? v[k] * __ldg(scale + k) : 0.f;
            mx = fmaxf(mx, v[k]);      // a NaN sum is dropped here and resurfaces through the scale below
          }
          const bool some = mx > 0.f;
          const float inv = some ? __frcp_rn(mx) : 0.f;
          float sc = some ? base + lg2f(mx) : NEG;
          if (base != base) sc = base;
          if (s.dest == kDualDestRoot) {
            sc = base;                 // a single sum: keep it unnormalised, its logarithm is taken by the fold
          } else {
#pragma unroll
            for (int k = 0; k < KMAX; ++k) v[k] *= inv;
          }
          deliver(s, v, sc);
        }
        PROF_ADD(P_W_DELIVER, tD);
        PROF_ADD(P_W_INNER, tI);
      }
      if (live && !failed) out[row] = (rootM + lg2f(rootS)) * 0x1.62e43p-1f;
    }
    PROF_ADD(P_W_TOTAL, tW);
  } else if (warp < 2 * 4 + NTILE) {
    // ================================ MMA issuers, one warp per tile =================================
    const unsigned t = warp - 2 * 4;
    const unsigned bT = t * BAR_TILE;
    const unsigned idescLeaf = (1u << 4) | ((unsigned)(KMAX >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
    const unsigned idescSum = (1u << 4) | ((unsigned)(NBLK >> 3) << 17) | ((unsigned)(TS >> 4) << 24);
    // Descriptors of the operand areas' first blocks, built once: a block further on adds its byte offset / 16
    // to the start-address field (the sum stays inside the field: shared memory ends below 256 KB).
    const unsigned long long aDesc = smemDesc(smemAddr(abuf) + t * A_TILE, KSTEP_A / 2, 128);
    const unsigned long long bDesc0 = smemDesc(smemAddr(bring), KSTEP_B / 2, 128);
    const unsigned long long lwDesc0 = smemDesc(smemAddr(lring), KSTEP_BL / 2, 128);
    const unsigned acc = tmem + t * 2 * NBLK;
    unsigned phOpReady = 0, phAccFree0 = 0, phAccFree1 = 0;
    unsigned wCount = 0;                // weight blocks consumed so far: ring slot and parity
    unsigned leafRing = 0, leafPar = 0; // ring slot and parity of the next leaf stage
    bool withheld = !(a.testWithholdCommit != 0 && t == 0);
    const long long tIs = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        const long long tStep = PROF_T();
        if (s.op == kLeafRegion) {
          const int nst = s.numBlocks;
#pragma unroll 1
          for (int st = 0; st < nst && !failed; ++st) {
            // the workers' arrival implies that the stage's weights have landed: they waited for the same
            // ring slot's barrier before they read their inputs from it
            const long long tq3 = PROF_T();
            if (!w.wait(bar(bT + BAR_LEAFFULL + (int)leafRing), leafPar)) { failed = true; break; }
            PROF_ADD(P_I_WAIT_LEAFFULL, tq3);
            if (lane == 0) {
              fenceAfter();
              const unsigned arows = acc + leafOperandCol(leafRing);   // operand rows written by the workers
              const unsigned long long lwd = lwDesc0 + (unsigned)((leafRing * LEAF_SLOT) >> 4);
#pragma unroll
              for (int ks = 0; ks < STAGE_FEATS / 2; ++ks)
                mmaF16TmemA(acc, arows + 8 * ks, lwd + (unsigned)((ks * KSTEP_BL) >> 4), idescLeaf, (st | ks) ? 1u : 0u);
              // one commit frees the ring slot for the loader and, through it, the operand rows for the workers
              mmaCommit(bar(BAR_LWEMPTY + (int)leafRing));
              if (st == nst - 1) mmaCommit(bar(BAR_LEAFDONE + t));
            }
            __syncwarp();
            if (++leafRing == (unsigned)LR) { leafRing = 0; leafPar ^= 1; }
          }
          PROF_ADD(P_I_LEAF, tStep);
          continue;
        }
        const int nblk = s.numBlocks;
#pragma unroll 1
        for (int nb = 0; nb < nblk && !failed; ++nb) {
          const unsigned ring = wCount % (unsigned)NB;
          const int b = nb & 1;
          if (nb == 0) {
            const long long tq4 = PROF_T();
            if (!w.wait(bar(bT + BAR_OPREADY), phOpReady)) { failed = true; break; }
            PROF_ADD(P_I_WAIT_OPREADY, tq4);
            phOpReady ^= 1;
          } else if (nb >= 2) {
            const long long tq5 = PROF_T();
            if (!w.wait(bar(bT + BAR_ACCFREE + b), b == 0 ? phAccFree0 : phAccFree1)) { failed = true; break; }
            PROF_ADD(P_I_WAIT_ACCFREE, tq5);
            if (b == 0) phAccFree0 ^= 1; else phAccFree1 ^= 1;
          }
          {
            const long long tq = PROF_T();
            if (!w.wait(bar(BAR_WFULL + ring), (wCount / (unsigned)NB) & 1)) { failed = true; break; }
            PROF_ADD(P_I_WAIT_WFULL, tq);
          }
          if (lane == 0) {
            fenceAfter();
            const unsigned d = acc + b * NBLK;
            const unsigned long long bdBlock = bDesc0 + (unsigned)((ring * B_BLOCK) >> 4);
            // value x value, residue x value, value x residue, each over j 0..15 and j 16..31
#pragma unroll
            for (int m = 0; m < 6; ++m) {
              const int aks = (m < 4) ? m : m - 4;   // A k-step: 0,1 value; 2,3 residue; 0,1 value
              const int bks = (m < 2) ? m : m - 2;   // B k-step: 0,1 value; 0,1 value; 2,3 residue
              mmaF16(d, aDesc + (unsigned)((aks * KSTEP_A) >> 4), bdBlock + (unsigned)((bks * KSTEP_B) >> 4), idescSum, m ? 1u : 0u);
            }
            // self-test: leave out one commit, so that the waits for it run out
            if (!withheld) withheld = true;
            else mmaCommit(bar(bT + BAR_ACCFULL + b));
            // the block's ring slot is free once both tiles' MMAs on it are done.  (A ring slot's own barrier
            // cannot run ahead of the loader that waits for it; the accumulator barriers can, by a whole phase
            // pair, so the loader does not wait on those.)
            mmaCommit(bar(BAR_WEMPTY + (int)ring));
          }
          __syncwarp();
          ++wCount;
        }
        PROF_ADD(P_I_INNER, tStep);
      }
    }
    PROF_ADD(P_I_TOTAL, tIs);
    // every MMA issued by this warp has completed when this barrier flips (also after a failure)
    if (lane == 0) mmaCommit(bar(BAR_DRAIN + t));
    __syncwarp();
    w.wait(bar(BAR_DRAIN + t), 0);
  } else if (warp == 2 * 4 + NTILE) {
    // ================================ inner-region weight loader =====================================
    unsigned issued = 0;
    const unsigned bAddr = smemAddr(bring);
    const long long tLs = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        if (s.op == kLeafRegion) continue;
        const unsigned char* src = a.frags + s.fragOffset;
        for (int nb = 0; nb < s.numBlocks && !failed; ++nb) {
          const unsigned ring = issued % (unsigned)NB;
          if (issued >= (unsigned)NB) {
            // the slot's previous block has been multiplied for both tiles
            const long long tq = PROF_T();
            if (!w.wait(bar(BAR_WEMPTY + ring), ((issued / (unsigned)NB) - 1) & 1)) { failed = true; break; }
            PROF_ADD(P_L_WAIT, tq);
          }
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
    // ================================ leaf loader: weights, inputs and centres of every stage ===========
    // Per stage of four features: 2 KB of weights, the four features' values for the 256 samples of the tile
    // pair (1 KB each, contiguous in the feature-major copy) and the four centres, all onto one barrier.
    unsigned issued = 0;
    const unsigned lAddr = smemAddr(lring);
    const long long tLs = PROF_T();
    for (unsigned long long pair = blockIdx.x; pair < npairs && !failed; pair += gridDim.x) {
      const float* xpair = xt + pair * (NTILE * TS);
      for (int si = 0; si < a.numSteps && !failed; ++si) {
        const DualStepDev s = a.steps[si];
        if (s.op != kLeafRegion) continue;
        const unsigned char* src = a.frags + s.fragOffset;
        for (int st = 0; st < s.numBlocks && !failed; ++st) {
          const unsigned ring = issued % (unsigned)LR;
          if (issued >= (unsigned)LR) {
            // both issuers' MMAs on the slot's previous stage are done (the workers read their inputs before)
            const long long tq = PROF_T();
            if (!w.wait(bar(BAR_LWEMPTY + ring), ((issued / (unsigned)LR) - 1) & 1)) { failed = true; break; }
            PROF_ADD(P_LL_WAIT, tq);
          }
          const unsigned dst = lAddr + ring * LEAF_SLOT;
          const unsigned full = bar(BAR_LWFULL + ring);
          if (lane == 0) mbarExpectTx(full, LEAF_SLOT_TX);
          __syncwarp();
          const int g = s.stageBase + st;
          if (lane == 0) bulkLoad(dst, src + (size_t)st * LW_STAGE, LW_STAGE, full);
          else if (lane <= STAGE_FEATS) bulkLoad(dst + LW_STAGE + (lane - 1) * (NTILE * TS * 4),
                                                 xpair + (size_t)__ldg(a.leafCols + g * STAGE_FEATS + (int)lane - 1) * a.xtLd,
                                                 NTILE * TS * 4, full);
          else if (lane == STAGE_FEATS + 1) bulkLoad(dst + LW_STAGE + LEAF_X, a.leafCentres + (size_t)g * STAGE_FEATS, STAGE_FEATS * 4, full);
          // (Asking rows of later stages into L2 ahead of time with cp.async.bulk.prefetch.L2 made the 2 M-sample
          // step slower, 221 ms against 201 ms: the tile pairs of all CTAs together are about as large as L2.)
          __syncwarp();
          ++issued;
        }
      }
    }
    PROF_ADD(P_LL_TOTAL, tLs);
    const unsigned pending = issued < (unsigned)LR ? issued : (unsigned)LR;
    for (unsigned i = issued - pending; i < issued; ++i) w.wait(bar(BAR_LWFULL + i % (unsigned)LR), (i / (unsigned)LR) & 1);
  }

  // ---- common exit: report, wait for the other roles' drains, free the tensor memory --------------------
  if (failed || *abortFlag) atomicExch(status, 1);
  if (PROFILE && profOn) {
    const int lo = tid == 0 ? 0 : (warp == 8 ? 16 : (warp == 10 ? 32 : 40)), hi = lo + (tid == 0 ? 16 : (warp == 8 ? 16 : 8));
    for (int i = lo; i < hi; ++i) profOut[i] = prof[i];
  }
  fenceBefore();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

size_t layeredDualGlobalStackBytes(int grid, int globalSlots) {
  return (size_t)grid * NTILE * (size_t)globalSlots * SLOT_FLOATS * 4;
}

size_t layeredDualSmemBytes(int aSlots, int ringBlocks, int leafRing) {
  return (size_t)NTILE * aSlots * SLOT_FLOATS * 4 + NTILE * A_TILE + (size_t)ringBlocks * B_BLOCK +
         (size_t)leafRing * LEAF_SLOT + NBARS * 8 + 16;
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
    cudaError_t e = a.foldScalar ? run(layeredDualKernel<true, false, true>, dProf) : run(layeredDualKernel<true, true, true>, dProf);
    long long h[P_COUNT];
    cudaMemcpy(h, dProf, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(dProf);
    static const char* names[P_COUNT] = {"w_total", "w_leaf", "w_leaf_wait_data", "w_leaf_wait_empty", "w_leaf_wait_done", "w_inner",
        "w_inner_prep", "w_inner_wait_full", "w_inner_fold", "w_deliver", "w_leaf_fence", "w_leaf_build", 0, 0, 0, 0,
        "i_total", "i_wait_opready", "i_wait_accfree", "i_wait_wfull", "i_wait_leaffull", "i_leaf", "i_inner", 0, 0, 0, 0, 0, 0, 0, 0, 0,
        "l_total", "l_wait", 0, 0, 0, 0, 0, 0, "ll_total", "ll_wait"};
    std::fprintf(stderr, "[dual profile] n=%zu grid=%d:", n, grid);
    for (int i = 0; i < P_COUNT; ++i) if (names[i]) std::fprintf(stderr, " %s=%lld", names[i], h[i]);
    std::fprintf(stderr, "\n");
    return e;
  }
  if (a.foldScalar) return a.marginal ? run(layeredDualKernel<true, false, false>, nullptr) : run(layeredDualKernel<false, false, false>, nullptr);
  return a.marginal ? run(layeredDualKernel<true, true, false>, nullptr) : run(layeredDualKernel<false, true, false>, nullptr);
}

}  // namespace spnb
