/*
 * spnb.h -- C ABI of the B200-native SPN joint log-likelihood engine (libspnb.so).
 *
 * This is the boundary a maintainer of the reference binds instead of the pieces listed beside
 * each entry point (paths are inside the reference project).  Plain pointers and sizes only;
 * every function returns 0 on success and a non-zero status otherwise, with a message available
 * from spnb_last_error() (thread-local).  No function throws across the boundary.
 *
 * Life cycle:   spnb_compile (needs no GPU)  ->  spnb_plan_load  ->  spnb_execute_*  ->  spnb_plan_free
 */
#ifndef SPNB_H
#define SPNB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct spnb_plan spnb_plan;

/* Field-for-field the metadata of the reference's kernel descriptor
 * (common/include/Kernel.h:39-126: queryType, target, batchSize, numFeatures, bytesPerFeature,
 * numResults, bytesPerResult, dtype). */
typedef struct spnb_kernel_info {
  char kernel_name[256];
  uint32_t query_type;        /* 1 = joint probability (common/include/Kernel.h:20) */
  uint32_t target;            /* 2 = CUDA (common/include/Kernel.h:22) */
  uint32_t batch_size;
  uint32_t num_features;
  uint32_t bytes_per_feature;
  uint32_t num_results;
  uint32_t bytes_per_result;
  char dtype[16];             /* result dtype: "float32" (log space) or "float64" (linear space) */
} spnb_kernel_info;

/* Status codes. */
enum {
  SPNB_OK = 0,
  SPNB_ERR_COMPILE = 1,       /* the reference throws std::runtime_error("COMPILATION ERROR") here */
  SPNB_ERR_RUNTIME = 2,       /* ... and std::runtime_error("RUNTIME ERROR") here */
  SPNB_ERR_ARGUMENT = 3,
  SPNB_ERR_CUDA = 4
};

/*
 * Compile an xspn query file into a plan file.
 * Replaces spnc::spn_compiler::compileQuery (compiler/include/spnc.h:22-48, compiler/src/Driver.cpp:22-44)
 * and everything behind it for the CUDA target (front end, lowering, cubin serialisation, linking:
 * compiler/src/toolchain/CUDAGPUToolchain.cpp:29-105).
 * Options are the reference's string->string option map (compiler/src/option/GlobalOptions.cpp:14-75);
 * unknown keys are an error, as in compiler/src/option/Options.h:222-224.  "target" must be "CUDA".
 * plan_out_path == NULL or "" lets the library pick a temporary file; the chosen path is returned in
 * plan_path_out (capacity plan_path_cap bytes).  Needs no GPU (NVRTC cross-compiles for sm_100a).
 */
int spnb_compile(const char* query_path, const char* const* opt_keys, const char* const* opt_vals, int n_opts,
                 const char* plan_out_path, char* plan_path_out, size_t plan_path_cap, spnb_kernel_info* info_out);

/* Load a plan file written by spnb_compile.  Replaces the dlopen/dlsym of the generated kernel
 * library (runtime/src/Executable.cpp:116-132).  Needs no GPU until the first execute. */
int spnb_plan_load(const char* plan_path, spnb_plan** plan_out);

int spnb_plan_info(const spnb_plan* plan, spnb_kernel_info* info_out);

/* JSON with the planner's statistics (nodes per kind, edges, depth, algorithmic ops and bytes per
 * sample, kernel strategy, registers).  Same role as the reference's graph statistics
 * (mlir/lib/Dialect/LoSPN/Passes/LoSPNGraphStatsCollection.cpp:83-102).  Valid until the plan is freed. */
const char* spnb_plan_stats_json(const spnb_plan* plan);

/* The CUDA C++ source generated for the plan ("" for the interpreter strategy); what "dump-ir" shows. */
const char* spnb_plan_source(const spnb_plan* plan);

/*
 * Evaluate n samples held in HOST memory: in = n x num_features x bytes_per_feature bytes, row-major,
 * C-contiguous; out = n x bytes_per_result bytes.  Returns after the results are in out.
 * Replaces spnc_rt::spn_runtime::execute -> Executable::executeGPU -> generated host stub
 * (runtime/src/runtime.cpp:42-49, runtime/src/Executable.cpp:105-114) and the mgpu* wrappers it
 * calls (runtime/wrappers/cuda/CUDARuntimeWrappers.cpp:56-153).  Runs on CUDA device 0 like the
 * reference unless spnb_set_device was called; copies are chunked and overlapped with compute.
 */
int spnb_execute_host(spnb_plan* plan, size_t n, const void* in, void* out);

/*
 * Evaluate n samples already resident in DEVICE memory of `device`, asynchronously on `cuda_stream`
 * (a cudaStream_t, NULL = default stream).  No counterpart in the reference, whose generated stub always
 * allocates and copies (mlir/lib/Conversion/LoSPNtoGPU/GPUStructurePatterns.cpp:81-100,142-146).
 */
int spnb_execute_device(spnb_plan* plan, int device, size_t n, const void* d_in, void* d_out, void* cuda_stream);

/*
 * Same contract as spnb_execute_device (device-resident in/out, asynchronous on cuda_stream), but nothing on
 * this path allocates or frees device memory.  It has no counterpart in the reference.  It is meant for
 * callers that may not allocate when they run a model: inside a latency-critical serving loop or any phase
 * where cudaMalloc's device-wide synchronisation is unacceptable, or under a fixed device-memory budget
 * agreed before start-up.  The model runs through the interpreter kernel (log-space plans only); the model
 * image and the kernel's spill scratch live in one 32 MiB device array that is part of the library itself,
 * so every GPU that loads the library gives up 32 MiB until the process exits.
 *   - Limit: the plan's image (op stream + leaf tables) plus one CTA's scratch must fit into the 32 MiB;
 *     otherwise the call fails with SPNB_ERR_RUNTIME and a message naming the limit.  n is not limited.
 *   - The first call on a device looks up the array's device address.  A call copies its plan's image into
 *     the array (cudaMemcpyAsync on cuda_stream) whenever another plan's image was the last one stored
 *     there, i.e. on the first call with a plan and again after every switch between plans.  Make such calls
 *     before any stream capture: while cuda_stream is capturing, a call that would have to replace the image
 *     fails with SPNB_ERR_RUNTIME instead.
 *   - The array is shared by all plans and calls of the process and keeps the previous call's contents;
 *     nothing in it has to be cleared.  Calls that overlap on the GPU (two streams, two threads) race on it:
 *     order them.  With two different plans the race is more than a wrong result: a kernel running one
 *     plan's program counts over the other plan's image can access memory outside its scratch.  For the
 *     same reason a launch recorded earlier stays valid only while its plan's image is still resident.
 */
int spnb_execute_device_noalloc(spnb_plan* plan, int device, size_t n, const void* d_in, void* d_out,
                                void* cuda_stream);

/*
 * Evaluate n host-resident samples on several GPUs of this process: the batch is split into contiguous
 * row blocks, one per listed device, the model tables are replicated on each device; no collective is
 * involved.  If mean_ll_out != NULL it receives the mean log-likelihood over all n samples (summed in
 * double on the host).  The reference runs on device 0 only (CUDARuntimeWrappers.cpp:36-54).
 */
int spnb_execute_sharded(spnb_plan* plan, const int* devices, int n_devices, size_t n, const void* in, void* out,
                         double* mean_ll_out);

/* Device used by spnb_execute_host (default 0). */
int spnb_set_device(spnb_plan* plan, int device);

/* Launch geometry the plan uses on `device`: CTAs, threads per CTA, dynamic shared memory bytes. */
int spnb_launch_config(spnb_plan* plan, int device, int* grid, int* block, size_t* smem_bytes);

/* Waits for the work this plan has queued on `device` (all streams) and reports whether a kernel gave up on
 * a bounded wait for the tensor cores (the tcgen05 layered kernel polls its barriers a limited number of
 * times and raises a flag instead of hanging).  spnb_execute_host checks the flag itself; after
 * spnb_execute_device, which returns before the kernel has run, this is the call that tells.  Returns 0 if
 * all results are complete.  No counterpart in the reference (its kernels have no such waits). */
int spnb_device_status(spnb_plan* plan, int device);

/* Milliseconds the kernel(s) of the last spnb_execute_host call took on the device (CUDA events). */
float spnb_last_kernel_ms(const spnb_plan* plan);

void spnb_plan_free(spnb_plan* plan);

/* Measured instruction rates of the current CUDA device, the compute denominators of the roofline:
 * kind 0 = FP32 fused multiply-adds per second, 1 = ex2.approx per second, 2 = lg2.approx per second,
 * 3 = FP64 fused multiply-adds per second, 4 = FP32 fused multiply-adds per second issued as packed pairs
 * (fma.rn.f32x2).  No counterpart in the reference (it has no measurement
 * code for the GPU path). */
int spnb_measure_peak(int kind, double* ops_per_second);

/* Number of CUDA devices visible (0 if there is no driver). Backs SPNCompiler.isTargetSupported("CUDA")
 * (compiler/src/Driver.cpp:47-59). */
int spnb_device_count(void);

const char* spnb_last_error(void);
const char* spnb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SPNB_H */
