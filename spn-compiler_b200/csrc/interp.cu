// Table-driven interpreter kernel for DAGs too large to unroll: one thread per sample, the op
// stream is walked by every thread in lock step (all control flow is warp-uniform), values live
// in shared-memory slots [slot][thread] assigned by liveness in the planner.
//
// Replaces what the reference does for oversized graphs, namely splitting the task into
// partitions with feature-major [k x N] intermediates in global memory
// (mlir/lib/Dialect/LoSPN/Passes/LoSPNTaskPartitioner.cpp:36-148); here intermediates never
// leave the SM.  Arithmetic is the same log-space formulation as the generated kernels: base-2
// logarithms, products are adds, sums are max-shifted log-sum-exp on the SFU.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "interp.h"

namespace spnb {

namespace {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ int toIntSat(T v);
template <> __device__ __forceinline__ int toIntSat<float>(float v) { return __float2int_rz(v); }
template <> __device__ __forceinline__ int toIntSat<double>(double v) { return __double2int_rz(v); }
template <> __device__ __forceinline__ int toIntSat<int8_t>(int8_t v) { return v; }
template <> __device__ __forceinline__ int toIntSat<uint8_t>(uint8_t v) { return v; }
template <> __device__ __forceinline__ int toIntSat<int16_t>(int16_t v) { return v; }
template <> __device__ __forceinline__ int toIntSat<uint16_t>(uint16_t v) { return v; }
template <> __device__ __forceinline__ int toIntSat<int32_t>(int32_t v) { return v; }
template <> __device__ __forceinline__ int toIntSat<uint32_t>(uint32_t v) { return v > 2147483647u ? 2147483647 : (int)v; }
template <> __device__ __forceinline__ int toIntSat<int64_t>(int64_t v) {
  return v > 2147483647ll ? 2147483647 : (v < -2147483648ll ? (-2147483647 - 1) : (int)v);
}
template <> __device__ __forceinline__ int toIntSat<uint64_t>(uint64_t v) { return v > 2147483647ull ? 2147483647 : (int)v; }

template <typename T> struct IsFloat { static constexpr bool value = false; };
template <> struct IsFloat<float> { static constexpr bool value = true; };
template <> struct IsFloat<double> { static constexpr bool value = true; };

// Shared memory: [fm int4 x F][xs real x NV*SX][cs u16 x NC*SX][pad to 8][vals real x nslots*TILE]
// LINEAR = false: values are base-2 logarithms in float (products add, sums are max-shifted log-sum-exp).
// LINEAR = true:  values are probabilities in double, one natural log at the root: the reference's f64 mode
// (mlir/lib/Conversion/HiSPNtoLoSPN/NodePatterns.cpp:140-151) for DAGs too large or too wide to unroll; the
// op stream then names its constants (Gaussian parameters, sum weights) by index into a table of doubles.
template <typename in_t, bool LINEAR>
__global__ void __launch_bounds__(1024) interpKernel(InterpArgs a, const in_t* __restrict__ in, void* __restrict__ outv,
                                                       unsigned long long n) {
  using real = typename std::conditional<LINEAR, double, float>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const unsigned tid = threadIdx.x;
  const unsigned TILE = blockDim.x;
  const unsigned SX = TILE + 1;
  const unsigned F = a.numFeatures;
  int4* fm = reinterpret_cast<int4*>(smem_raw);
  real* xs = reinterpret_cast<real*>(smem_raw + (size_t)F * 16);
  unsigned short* cs = reinterpret_cast<unsigned short*>(xs + (size_t)a.numValueSlots * SX);
  real* vals = reinterpret_cast<real*>(smem_raw + a.valsOffset(TILE));
  for (unsigned i = tid; i < F; i += TILE) fm[i] = a.featureMeta[i];
  const int* __restrict__ prog = a.prog;
  const real* __restrict__ tab = static_cast<const real*>(a.tab);
  const double* __restrict__ dc = a.dconst;
  const unsigned char* __restrict__ lut = a.lut;
  const int* __restrict__ brk = a.breaks;
  const bool marginal = a.marginal != 0;
  real* out = static_cast<real*>(outv);

  const unsigned long long ntiles = (n + TILE - 1) / TILE;
  for (unsigned long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const unsigned long long base = tile * TILE;
    const unsigned rows = (n - base) < (unsigned long long)TILE ? (unsigned)(n - base) : TILE;
    __syncthreads();
    {
      const in_t* __restrict__ src = in + base * F;
      const unsigned total = rows * F;
      unsigned r = tid / F, c = tid - r * F;          // element e = tid + i*TILE -> (row, column)
      const unsigned dr = TILE / F, dcol = TILE - dr * F;
      for (unsigned e = tid; e < TILE * F; e += TILE) {
        const int4 m = fm[c];
        const bool live = e < total;
        in_t raw = 0;
        if (live) raw = src[e];
        if (m.w >= 0) xs[m.w * SX + r] = (real)raw;
        if (m.z >= 0) {
          const unsigned rr = (unsigned)toIntSat<in_t>(raw) - (unsigned)m.x;
          int code = rr < (unsigned)m.y ? (int)rr + 2 : 1;
          if (IsFloat<in_t>::value && raw != raw) code = 0;
          cs[m.z * SX + r] = (unsigned short)(live ? code : 1);
        }
        r += dr; c += dcol;
        if (c >= F) { c -= F; r += 1; }
      }
    }
    __syncthreads();
    const real* xcol = xs + tid;
    const unsigned short* ccol = cs + tid;
    real* v = vals + tid;
    // value slots: ids below numSlots are shared memory, the rest this CTA's part of the scratch area
    const int S = a.numSlots;
    real* g = static_cast<real*>(a.scratch) + ((size_t)blockIdx.x * a.numSpillSlots * TILE + tid);
    auto ld = [&](int s) -> real { return s < S ? v[s * TILE] : g[(size_t)(s - S) * TILE]; };
    int pc = 0;
    // the walk is bounded by the program length: a corrupt stream ends the tile instead of spinning
    while (pc < a.progLen) {
      const int op = __ldg(prog + pc);
      if (op == OP_END) {
        const real root = ld(__ldg(prog + pc + 1));
        if (tid < rows) {
          if (LINEAR) out[base + tid] = (real)log((double)root);
          else out[base + tid] = root * (real)0x1.62e43p-1f;
        }
        break;
      }
      const int dst = __ldg(prog + pc + 1);
      real r;
      switch (op) {
        case OP_GAUSS: {
          const real x = xcol[__ldg(prog + pc + 2) * SX];
          if (LINEAR) {
            const double d = (double)x - __ldg(dc + __ldg(prog + pc + 3));
            r = (real)(__ldg(dc + __ldg(prog + pc + 5)) * exp((d * d) * __ldg(dc + __ldg(prog + pc + 4))));
            if (marginal && d != d) r = (real)1;
          } else {
            const float d = (float)x - __int_as_float(__ldg(prog + pc + 3));
            r = (real)fmaf(d * d, __int_as_float(__ldg(prog + pc + 4)), __int_as_float(__ldg(prog + pc + 5)));
            if (marginal && d != d) r = (real)0;
          }
          pc += 6;
          break;
        }
        case OP_TABLE: {
          int code = ccol[__ldg(prog + pc + 2) * SX];
          const int lo = __ldg(prog + pc + 3);
          if (lo >= 0) code = __ldg(lut + lo + code);
          r = __ldg(tab + __ldg(prog + pc + 4) + code);
          pc += 5;
          break;
        }
        case OP_HISTG: {
          const real x = xcol[__ldg(prog + pc + 2) * SX];
          const int* b = brk + __ldg(prog + pc + 3);
          const int cnt = __ldg(prog + pc + 4);
          const int xi = LINEAR ? __double2int_rz((double)x) : __float2int_rz((float)x);
          int idx = cnt;
          if (xi >= __ldg(b) && xi < __ldg(b + cnt)) {
            idx = 0;
            for (int i = 1; i < cnt; ++i) idx += (xi >= __ldg(b + i));
          }
          if (x != x) idx = cnt + 1;
          r = __ldg(tab + __ldg(prog + pc + 5) + idx);
          pc += 6;
          break;
        }
        case OP_PROD: {
          const int k = min(__ldg(prog + pc + 2), a.progLen - pc);
          const int* s = prog + pc + 3;
          if (LINEAR) {
            real a0 = (real)1, a1 = (real)1;
            int i = 0;
            for (; i + 1 < k; i += 2) {
              a0 *= ld(__ldg(s + i));
              a1 *= ld(__ldg(s + i + 1));
            }
            if (i < k) a0 *= ld(__ldg(s + i));
            r = a0 * a1;
          } else {
            real a0 = (real)0, a1 = (real)0;
            int i = 0;
            for (; i + 1 < k; i += 2) {
              a0 += ld(__ldg(s + i));
              a1 += ld(__ldg(s + i + 1));
            }
            if (i < k) a0 += ld(__ldg(s + i));
            r = a0 + a1;
          }
          pc += 3 + k;
          break;
        }
        case OP_SUM: {
          const int k = min(__ldg(prog + pc + 2), (a.progLen - pc) / 2);
          const int* s = prog + pc + 3;
          if (LINEAR) {
            double acc0 = 0.0, acc1 = 0.0;
            int i = 0;
            for (; i + 1 < k; i += 2) {
              acc0 = fma(__ldg(dc + __ldg(s + 2 * i + 1)), (double)ld(__ldg(s + 2 * i)), acc0);
              acc1 = fma(__ldg(dc + __ldg(s + 2 * i + 3)), (double)ld(__ldg(s + 2 * i + 2)), acc1);
            }
            if (i < k) acc0 = fma(__ldg(dc + __ldg(s + 2 * i + 1)), (double)ld(__ldg(s + 2 * i)), acc0);
            r = (real)(acc0 + acc1);
          } else {
            float m = __int_as_float(0xff800000);
            for (int i = 0; i < k; ++i) m = fmaxf(m, (float)ld(__ldg(s + 2 * i)) + __int_as_float(__ldg(s + 2 * i + 1)));
            const float mm = (m == __int_as_float(0xff800000)) ? 0.0f : m;
            float acc0 = 0.0f, acc1 = 0.0f;
            int i = 0;
            for (; i + 1 < k; i += 2) {
              acc0 += ex2((float)ld(__ldg(s + 2 * i)) + __int_as_float(__ldg(s + 2 * i + 1)) - mm);
              acc1 += ex2((float)ld(__ldg(s + 2 * i + 2)) + __int_as_float(__ldg(s + 2 * i + 3)) - mm);
            }
            if (i < k) acc0 += ex2((float)ld(__ldg(s + 2 * i)) + __int_as_float(__ldg(s + 2 * i + 1)) - mm);
            r = (real)(m + lg2(acc0 + acc1));
          }
          pc += 3 + 2 * k;
          break;
        }
        default:  // unknown opcode: stop walking
          pc = a.progLen;
          continue;
      }
      if (dst < S) v[dst * TILE] = r;
      else g[(size_t)(dst - S) * TILE] = r;
    }
  }
}

template <typename in_t>
cudaError_t launchT(const InterpArgs& a, const void* in, void* out, size_t n, int grid, int tile, size_t smem,
                    cudaStream_t stream) {
  if (a.linear) {
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&interpKernel<in_t, true>), smem);
    if (e != cudaSuccess) return e;
    interpKernel<in_t, true><<<grid, tile, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n);
    return cudaGetLastError();
  }
  cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&interpKernel<in_t, false>), smem);
  if (e != cudaSuccess) return e;
  interpKernel<in_t, false><<<grid, tile, smem, stream>>>(a, static_cast<const in_t*>(in), out, (unsigned long long)n);
  return cudaGetLastError();
}

}  // namespace

size_t interpSmemBytes(const InterpArgs& a, int tile) {
  return a.valsOffset((unsigned)tile) + (size_t)a.numSlots * tile * (a.linear ? 8 : 4);
}

cudaError_t interpOccupancy(int inKindCode, int tile, size_t smem, int* blocksPerSM, bool linear) {
  // all instantiations have the same resource usage up to the staging conversion; query the float-input ones
  (void)inKindCode;
  if (linear) {
    cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&interpKernel<float, true>), smem);
    if (e != cudaSuccess) return e;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocksPerSM, interpKernel<float, true>, tile, smem);
  }
  cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(&interpKernel<float, false>), smem);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocksPerSM, interpKernel<float, false>, tile, smem);
}

cudaError_t interpLaunch(const InterpArgs& a, int dtypeCode, const void* in, void* out, size_t n, int grid, int tile,
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

// =========================================================================================================
// Interpreter without device allocations.
//
// Some callers must not allocate device memory at the time they run a model: a latency-critical serving
// loop (cudaMalloc synchronises the whole device), and hosts that hand this library a fixed memory budget
// up front.  For them the interpreter
// can run with everything it needs besides the caller's input and output buffers placed in one
// file-scope device array: first the model image (op stream, leaf tables, byte tables, breaks, feature
// descriptors), then the per-CTA spill scratch.  The array's size is fixed (kStaticAreaBytes); a model
// whose image plus one CTA's scratch does not fit is rejected.  The grid shrinks, if necessary, to as
// many CTAs as the scratch left over can serve.
//
// The array is shared by every call in the process and keeps whatever the last call left in it.  Nothing
// in it needs to start at zero: the image is rewritten when a different plan ran last, and every scratch
// slot is written before it is read within one tile.  Two calls that overlap on the GPU (different
// streams, or different host threads) race on it: callers must order them.  The race is not benign when the
// calls belong to different plans: a kernel launched with one plan's counts would then walk the other
// plan's op stream, whose slot and table indices it does not re-check, and may read or write outside its
// scratch.  Which image is resident is tracked on the host when a call is enqueued; a launch that is
// replayed later (a captured stream) is only valid while its plan's image is still the resident one, so an
// image swap is refused while the stream is capturing.
// =========================================================================================================
namespace {

static __device__ __align__(256) unsigned char g_staticArea[kStaticAreaBytes];

struct StaticAreaState {
  unsigned char* base = nullptr;      // device address of g_staticArea on this device
  unsigned long long resident = 0;    // tag of the image currently stored there
};
StaticAreaState g_areaState[64];
std::mutex g_areaMutex;

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

cudaError_t interpLaunchStatic(const InterpImage& img, InterpArgs a, int dtypeCode, const void* in, float* out, size_t n,
                               int tile, int device, cudaStream_t stream, const char** message) {
  if (message) *message = nullptr;
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_areaMutex);
  StaticAreaState& st = g_areaState[device];
  if (!st.base) {
    // In host code the array's name is only a handle; the kernel needs the address on this device.
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_staticArea);
    if (e != cudaSuccess) return e;
    st.base = static_cast<unsigned char*>(p);
  }
  const size_t offProg = 0;
  const size_t offTab = offProg + align256(img.progBytes);
  const size_t offLut = offTab + align256(img.tabBytes);
  const size_t offBrk = offLut + align256(img.lutBytes);
  const size_t offMeta = offBrk + align256(img.breaksBytes);
  const size_t offScratch = offMeta + align256(img.metaBytes);
  const size_t perCta = (size_t)a.numSpillSlots * (size_t)tile * sizeof(float);
  if (offScratch + perCta > kStaticAreaBytes) {
    if (message) *message = "model image and one CTA of spill scratch exceed the static device area (32 MiB)";
    return cudaErrorInvalidValue;
  }
  if (st.resident != img.tag) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      if (message) *message = "another plan's image is resident in the static device area and cannot be replaced while "
                              "the stream is capturing: run this plan once before the capture";
      return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaSuccess;
    auto put = [&](size_t off, const void* src, size_t bytes) {
      if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(st.base + off, src, bytes, cudaMemcpyHostToDevice, stream);
    };
    put(offProg, img.prog, img.progBytes);
    put(offTab, img.tab, img.tabBytes);
    put(offLut, img.lut, img.lutBytes);
    put(offBrk, img.breaks, img.breaksBytes);
    put(offMeta, img.meta, img.metaBytes);
    if (e != cudaSuccess) { st.resident = 0; return e; }
    st.resident = img.tag;
  }
  a.prog = reinterpret_cast<const int*>(st.base + offProg);
  a.tab = st.base + offTab;
  a.lut = st.base + offLut;
  a.breaks = reinterpret_cast<const int*>(st.base + offBrk);
  a.featureMeta = reinterpret_cast<const int4*>(st.base + offMeta);
  a.scratch = reinterpret_cast<float*>(st.base + offScratch);
  const size_t smem = interpSmemBytes(a, tile);
  int perSM = 0, sms = 0;
  cudaError_t e = interpOccupancy(dtypeCode, tile, smem, &perSM, false);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return e;
  if (perSM < 1) {
    if (message) *message = "interpreter kernel does not fit on one SM with this tile";
    return cudaErrorInvalidValue;
  }
  size_t grid = (size_t)perSM * (size_t)sms;
  if (perCta) grid = std::min(grid, (kStaticAreaBytes - offScratch) / perCta);
  const size_t tiles = (n + (size_t)tile - 1) / (size_t)tile;
  grid = std::min(grid, tiles);
  if (grid == 0) return cudaSuccess;
  return interpLaunch(a, dtypeCode, in, out, n, (int)grid, tile, smem, stream);
}

}  // namespace spnb
