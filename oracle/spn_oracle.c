/*
 * TEST INFRASTRUCTURE (oracle) -- CPU restatement of the reference's joint log-likelihood
 * arithmetic.  Only the tests, the smoke check and the CPU-baseline leg of the benchmark use
 * this file; the product never links, loads or calls it.
 *
 * What it restates (paths inside the reference project):
 *   - n-ary product / weighted sum -> balanced binary trees, left half = first ceil(k/2)
 *     operands, weight applied to each addend first:
 *       mlir/lib/Conversion/HiSPNtoLoSPN/NodePatterns.cpp:17-40 (product), :49-88 (sum)
 *   - root log in linear mode: NodePatterns.cpp:140-151
 *   - log-space arithmetic on the GPU: product = add, sum = a + log(1 + exp(b - a)) with
 *     a = (x > y ? x : y):  mlir/lib/Conversion/LoSPNtoGPU/GPUNodePatterns.cpp:164-179, :198-226
 *   - log-space sum on the CPU: a + log1p(exp(b - a)):
 *       mlir/lib/Conversion/LoSPNtoCPU/NodePatterns.cpp:216-240
 *   - Gaussian leaf, log: coef + (x-mu)^2 * d, coef = -ln(sigma) - 0.5 ln(2 pi), d = -1/(2 sigma^2),
 *     constants folded in double and rounded to the compute type; NaN -> 0 when marginal:
 *       GPUNodePatterns.cpp:292-360;  linear: coef' * exp((x-mu)^2 * d), NaN -> 1: :228-290
 *   - Categorical leaf: select chain over ln p_i, default -inf (log) / 0 (linear): :362-409
 *   - Histogram leaf: bucket i = [breaks[i], breaks[i+1]) -> ln density_i, outside -inf: :411-509
 *   - compute type: log-space is always f32, linear is f64:
 *       mlir/lib/Conversion/HiSPNtoLoSPN/HiSPNtoLoSPNConversionPasses.cpp:34-41
 *   - batching: chunks of samples distributed by an OpenMP parallel-for, SIMD across samples:
 *       runtime/src/Executable.cpp:83-103,
 *       mlir/lib/Conversion/LoSPNtoCPU/Vectorization/VectorizeStructurePatterns.cpp:325-423
 *
 * Deliberate choices where the reference is undefined or buggy (same as the product):
 *   - a sum whose addends are all -inf yields -inf; with strict_nan != 0 it yields NaN like the
 *     reference's b - a = (-inf) - (-inf);
 *   - a floating input is truncated toward zero to a signed 64-bit index for discrete leaves
 *     (the reference's fptoui of a negative value is undefined);
 *   - integer inputs keep the signedness of the declared numpy dtype.
 *
 * Parity status: pinned.  tests/test_oracle_golden.py checks this file against the reference's
 * stored model/input/output triples (NIPS5, nltcs, plants), the twelve known answers in
 * execute/src/main.cpp:32-52 and the f32 constants in
 * mlir/test/lowering/lospn-to-cpu/lower-to-cpu-nodes-scalar-log.mlir:206-213,340-349.
 *
 * This translation unit is compiled twice: plain (scalar libm, the checker) and with
 * -DORACLE_VECMATH (glibc libmvec SIMD exp/log/log1p, the timed CPU baseline).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifdef ORACLE_VECMATH
#define FN(name) name##_vec
/* glibc only attaches the SIMD variants under -ffast-math; that flag would also drop NaN/inf
 * semantics, so the vector variants are declared here instead. */
#pragma omp declare simd notinbranch
extern float expf(float);
#pragma omp declare simd notinbranch
extern float logf(float);
#pragma omp declare simd notinbranch
extern float log1pf(float);
#pragma omp declare simd notinbranch
extern double exp(double);
#pragma omp declare simd notinbranch
extern double log(double);
#pragma omp declare simd notinbranch
extern double log1p(double);
#else
#define FN(name) name
#endif

enum { K_PRODUCT = 0, K_SUM = 1, K_HIST = 2, K_GAUSS = 3, K_CAT = 4 };
enum { MODE_LINEAR_F64 = 0, MODE_LOG_F64_NARY = 1, MODE_LOG_F32_GPU = 2, MODE_LOG_F32_CPU = 3,
       MODE_LOG_F64_REFORDER = 4, MODE_LINEAR_F32 = 5 };
enum { DT_U8, DT_I8, DT_U16, DT_I16, DT_U32, DT_I32, DT_U64, DT_I64, DT_F32, DT_F64 };

typedef struct {
  int32_t n_nodes;
  int32_t root;
  int32_t num_features;
  int32_t pad_;
  const int32_t* kind;
  const int32_t* feature;
  const double* mean;
  const double* stddev;
  const int64_t* child_ptr;
  const int32_t* child_idx;
  const double* weights;
  const int64_t* tab_ptr;
  const double* tab;
  const int64_t* brk_ptr;
  const int32_t* brk;
} spn_model_t;

#define CH 256
#define MAXDEPTH 40

static int dt_is_float(int dt) { return dt >= DT_F32; }

/* one input element as double (exact for every supported type except |int64| > 2^53) */
static inline double load_as_double(const void* in, int dt, size_t idx) {
  switch (dt) {
    case DT_U8: return ((const uint8_t*)in)[idx];
    case DT_I8: return ((const int8_t*)in)[idx];
    case DT_U16: return ((const uint16_t*)in)[idx];
    case DT_I16: return ((const int16_t*)in)[idx];
    case DT_U32: return ((const uint32_t*)in)[idx];
    case DT_I32: return ((const int32_t*)in)[idx];
    case DT_U64: return (double)((const uint64_t*)in)[idx];
    case DT_I64: return (double)((const int64_t*)in)[idx];
    case DT_F32: return ((const float*)in)[idx];
    default: return ((const double*)in)[idx];
  }
}

/* slot plan shared by all chunks */
typedef struct {
  int n_order;
  int* order;   /* reachable nodes, children before parents */
  int* slot;    /* per node */
  int n_slots;
} plan_t;

static int build_plan(const spn_model_t* m, plan_t* p) {
  int n = m->n_nodes;
  char* reach = (char*)calloc(n, 1);
  int* stack = (int*)malloc(sizeof(int) * (size_t)(n + 1));
  int* uses = (int*)calloc(n, sizeof(int));
  p->order = (int*)malloc(sizeof(int) * (size_t)n);
  p->slot = (int*)malloc(sizeof(int) * (size_t)n);
  int sp = 0;
  stack[sp++] = m->root;
  reach[m->root] = 1;
  while (sp) {
    int v = stack[--sp];
    for (int64_t e = m->child_ptr[v]; e < m->child_ptr[v + 1]; ++e) {
      int c = m->child_idx[e];
      if (c >= v) { free(reach); free(stack); free(uses); return -1; } /* not children-first */
      uses[c]++;
      if (!reach[c]) { reach[c] = 1; stack[sp++] = c; }
    }
  }
  p->n_order = 0;
  for (int v = 0; v < n; ++v) if (reach[v]) p->order[p->n_order++] = v;
  /* free-list slot assignment in evaluation order */
  int* freel = stack;
  int nfree = 0, nslots = 0;
  for (int i = 0; i < p->n_order; ++i) {
    int v = p->order[i];
    int s = nfree ? freel[--nfree] : nslots++;
    p->slot[v] = s;
    for (int64_t e = m->child_ptr[v]; e < m->child_ptr[v + 1]; ++e) {
      int c = m->child_idx[e];
      if (--uses[c] == 0) freel[nfree++] = p->slot[c];
    }
  }
  p->n_slots = nslots;
  free(reach); free(stack); free(uses);
  return 0;
}

/* ---------------- generic body, instantiated for float and double ---------------- */
#define REAL float
#define SUF f32
#define R_EXP expf
#define R_LOG logf
#define R_LOG1P log1pf
#include "spn_oracle_body.inc"
#undef REAL
#undef SUF
#undef R_EXP
#undef R_LOG
#undef R_LOG1P

#define REAL double
#define SUF f64
#define R_EXP exp
#define R_LOG log
#define R_LOG1P log1p
#include "spn_oracle_body.inc"
#undef REAL
#undef SUF
#undef R_EXP
#undef R_LOG
#undef R_LOG1P

/*
 * Evaluate n samples (row-major [n x num_features] of in_dtype) and write n results of the
 * mode's compute type (float for the f32 modes, double otherwise).  threads <= 0: all cores.
 * chunk = samples per OpenMP work item (the reference's CPU batch size, default 4096).
 * Returns 0, or a negative code: -1 nodes not children-first, -2 bad arguments.
 */
int FN(spn_oracle_eval)(const spn_model_t* m, int mode, int marginal, int strict_nan, int in_dtype,
                        const void* in, size_t n, void* out, int threads, int chunk) {
  if (!m || in_dtype < 0 || in_dtype > DT_F64) return -2;
  if (marginal && !dt_is_float(in_dtype)) return -3; /* HiSPNOps.cpp:33-41 */
  plan_t p;
  if (build_plan(m, &p)) return -1;
  if (chunk <= 0) chunk = 4096;
#ifdef _OPENMP
  if (threads <= 0) threads = omp_get_max_threads();
#else
  threads = 1;
#endif
  int is32 = (mode == MODE_LOG_F32_GPU || mode == MODE_LOG_F32_CPU || mode == MODE_LINEAR_F32);
  size_t nchunks = (n + (size_t)chunk - 1) / (size_t)chunk;
  int rc = 0;
#pragma omp parallel num_threads(threads)
  {
    void* ws = is32 ? ws_alloc_f32(&p) : ws_alloc_f64(&p);
    if (!ws) {
#pragma omp atomic write
      rc = -4;
    }
#pragma omp for schedule(dynamic, 1)
    for (size_t c = 0; c < nchunks; ++c) {
      if (!ws) continue;
      size_t s0 = c * (size_t)chunk;
      size_t s1 = s0 + (size_t)chunk < n ? s0 + (size_t)chunk : n;
      for (size_t s = s0; s < s1; s += CH) {
        int cnt = (int)(s1 - s < CH ? s1 - s : CH);
        if (is32)
          eval_block_f32(m, &p, ws, mode, marginal, strict_nan, in_dtype, in, s, cnt, (float*)out + s);
        else
          eval_block_f64(m, &p, ws, mode, marginal, strict_nan, in_dtype, in, s, cnt, (double*)out + s);
      }
    }
    if (is32) ws_free_f32(ws); else ws_free_f64(ws);
  }
  free(p.order);
  free(p.slot);
  return rc;
}

int FN(spn_oracle_max_threads)(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
