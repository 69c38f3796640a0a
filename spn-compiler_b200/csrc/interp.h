// Launch interface of the interpreter kernel (interp.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <utility>

#include "plan.h"

namespace spnb {

// input element types, in the order the C-ABI documents them
enum DTypeCode : int { DT_U8 = 0, DT_I8, DT_U16, DT_I16, DT_U32, DT_I32, DT_U64, DT_I64, DT_F32, DT_F64 };

struct InterpArgs {
  const int* prog;              // device: op stream
  const void* tab;              // device: leaf tables (float, log2 domain; double probabilities in linear mode)
  const double* dconst;         // device: linear mode: the constants the op stream refers to by index
  const unsigned char* lut;     // device: code -> bucket byte tables
  const int* breaks;            // device: breaks of the generic histogram groups
  const int4* featureMeta;      // device: per feature (lo, domain, codeSlot, valueSlot)
  int progLen;                  // number of int32 words in prog
  int numFeatures;
  int numValueSlots;
  int numCodeSlots;
  int numSlots;                 // value slots in shared memory
  int numSpillSlots;            // value slots in the scratch area
  void* scratch;                // device: [grid][numSpillSlots][tile] values, or null
  int marginal;
  int linear;                   // 1: linear-space f64 evaluation with one log at the root (values are doubles)
  // byte offset of the value slots behind the staged inputs for a CTA of `tile` threads
  __host__ __device__ size_t valsOffset(unsigned tile) const {
    size_t sx = (size_t)tile + 1;
    size_t rb = linear ? 8 : 4;
    size_t o = (size_t)numFeatures * 16 + (size_t)numValueSlots * sx * rb + (size_t)numCodeSlots * sx * 2;
    return (o + 7) & ~(size_t)7;
  }
};

// Raises a kernel's dynamic shared-memory limit to `smem` bytes on the current device.  The attribute is
// per device and per function and only ever needs to grow, so the driver is called the first time and when
// a larger size is asked for, not on every launch.
inline cudaError_t ensureDynamicSmem(const void* kernel, size_t smem) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, size_t> granted;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  size_t& have = granted[std::make_pair(device, kernel)];
  if (smem <= have || smem <= 48 * 1024) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) have = smem;
  return e;
}

size_t interpSmemBytes(const InterpArgs& a, int tile);
cudaError_t interpOccupancy(int dtypeCode, int tile, size_t smem, int* blocksPerSM, bool linear);
cudaError_t interpLaunch(const InterpArgs& a, int dtypeCode, const void* in, void* out, size_t n, int grid, int tile,
                         size_t smem, cudaStream_t stream);

// ---- variant without device allocations ---------------------------------------------------------------
// Size of the file-scope device area that holds the model image and the spill scratch of
// interpLaunchStatic.  Every GPU that loads the library keeps this much memory until the process exits.
constexpr size_t kStaticAreaBytes = 32u << 20;

// Host copies of everything the interpreter reads on the device besides inputs and outputs.
struct InterpImage {
  const void* prog = nullptr;   size_t progBytes = 0;
  const void* tab = nullptr;    size_t tabBytes = 0;
  const void* lut = nullptr;    size_t lutBytes = 0;
  const void* breaks = nullptr; size_t breaksBytes = 0;
  const void* meta = nullptr;   size_t metaBytes = 0;
  unsigned long long tag = 0;   // identifies the image; a different tag forces a new upload
};

// Runs the interpreter with its model image and spill scratch inside the static device area: no
// cudaMalloc / cudaFree anywhere on this path.  `a` carries the counts (pointers are filled in here).
// Returns cudaSuccess or an error; *message (if not null) receives a static explanation for
// capacity errors.
cudaError_t interpLaunchStatic(const InterpImage& img, InterpArgs a, int dtypeCode, const void* in, float* out, size_t n,
                               int tile, int device, cudaStream_t stream, const char** message);

}  // namespace spnb
