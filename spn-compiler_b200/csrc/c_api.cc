// extern "C" surface of libspnb.so (declared in include/spnb.h): status codes instead of exceptions.
#include <cuda_runtime.h>

#include <cstring>
#include <string>

#include "../../include/spnb.h"
#include "engine.h"

using namespace spnb;

struct spnb_plan {
  std::unique_ptr<Engine> engine;
};

namespace {
thread_local std::string g_lastError;

void fillInfo(const KernelMeta& m, spnb_kernel_info* info) {
  if (!info) return;
  std::memset(info, 0, sizeof(*info));
  std::strncpy(info->kernel_name, m.kernelName.c_str(), sizeof(info->kernel_name) - 1);
  info->query_type = m.queryType;
  info->target = m.target;
  info->batch_size = m.batchSize;
  info->num_features = m.numFeatures;
  info->bytes_per_feature = m.bytesPerFeature;
  info->num_results = m.numResults;
  info->bytes_per_result = m.bytesPerResult;
  std::strncpy(info->dtype, m.dtype.c_str(), sizeof(info->dtype) - 1);
}

template <typename Fn>
int guarded(int errCode, Fn&& fn) {
  try {
    fn();
    return SPNB_OK;
  } catch (const std::exception& e) {
    g_lastError = e.what();
    return g_lastError.rfind("CUDA", 0) == 0 ? SPNB_ERR_CUDA : errCode;
  } catch (...) {
    g_lastError = "unknown error";
    return errCode;
  }
}
}  // namespace

extern "C" {

int spnb_compile(const char* query_path, const char* const* opt_keys, const char* const* opt_vals, int n_opts,
                 const char* plan_out_path, char* plan_path_out, size_t plan_path_cap, spnb_kernel_info* info_out) {
  if (!query_path || n_opts < 0 || (n_opts > 0 && (!opt_keys || !opt_vals))) {
    g_lastError = "spnb_compile: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_COMPILE, [&] {
    std::vector<std::pair<std::string, std::string>> kv;
    for (int i = 0; i < n_opts; ++i) kv.emplace_back(opt_keys[i] ? opt_keys[i] : "", opt_vals[i] ? opt_vals[i] : "");
    Options opt = parseOptions(kv);
    KernelMeta meta;
    std::string path = Engine::compile(query_path, opt, plan_out_path ? plan_out_path : "", &meta);
    if (plan_path_out && plan_path_cap) {
      if (path.size() + 1 > plan_path_cap) throw std::runtime_error("plan path buffer too small");
      std::memcpy(plan_path_out, path.c_str(), path.size() + 1);
    }
    fillInfo(meta, info_out);
  });
}

int spnb_plan_load(const char* plan_path, spnb_plan** plan_out) {
  if (!plan_path || !plan_out) {
    g_lastError = "spnb_plan_load: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  *plan_out = nullptr;
  return guarded(SPNB_ERR_RUNTIME, [&] {
    std::unique_ptr<spnb_plan> p(new spnb_plan());
    p->engine = Engine::load(plan_path);
    *plan_out = p.release();
  });
}

int spnb_plan_info(const spnb_plan* plan, spnb_kernel_info* info_out) {
  if (!plan || !info_out) {
    g_lastError = "spnb_plan_info: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  fillInfo(plan->engine->meta(), info_out);
  return SPNB_OK;
}

const char* spnb_plan_stats_json(const spnb_plan* plan) { return plan ? plan->engine->statsJson().c_str() : ""; }
const char* spnb_plan_source(const spnb_plan* plan) { return plan ? plan->engine->source().c_str() : ""; }

int spnb_execute_host(spnb_plan* plan, size_t n, const void* in, void* out) {
  if (!plan || (n && (!in || !out))) {
    g_lastError = "spnb_execute_host: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME, [&] { plan->engine->executeHost(n, in, out); });
}

int spnb_execute_device(spnb_plan* plan, int device, size_t n, const void* d_in, void* d_out, void* cuda_stream) {
  if (!plan || (n && (!d_in || !d_out))) {
    g_lastError = "spnb_execute_device: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME, [&] { plan->engine->executeDevice(device, n, d_in, d_out, (cudaStream_t)cuda_stream); });
}

int spnb_execute_device_noalloc(spnb_plan* plan, int device, size_t n, const void* d_in, void* d_out, void* cuda_stream) {
  if (!plan || (n && (!d_in || !d_out))) {
    g_lastError = "spnb_execute_device_noalloc: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME,
                 [&] { plan->engine->executeDeviceNoAlloc(device, n, d_in, d_out, (cudaStream_t)cuda_stream); });
}

int spnb_execute_sharded(spnb_plan* plan, const int* devices, int n_devices, size_t n, const void* in, void* out,
                         double* mean_ll_out) {
  if (!plan || !devices || n_devices <= 0 || (n && (!in || !out))) {
    g_lastError = "spnb_execute_sharded: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME, [&] { plan->engine->executeSharded(devices, n_devices, n, in, out, mean_ll_out); });
}

int spnb_set_device(spnb_plan* plan, int device) {
  if (!plan || device < 0) {
    g_lastError = "spnb_set_device: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  plan->engine->setDevice(device);
  return SPNB_OK;
}

int spnb_launch_config(spnb_plan* plan, int device, int* grid, int* block, size_t* smem_bytes) {
  if (!plan) {
    g_lastError = "spnb_launch_config: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME, [&] { plan->engine->launchConfig(device, grid, block, smem_bytes); });
}

int spnb_device_status(spnb_plan* plan, int device) {
  if (!plan) {
    g_lastError = "spnb_device_status: invalid argument";
    return SPNB_ERR_ARGUMENT;
  }
  return guarded(SPNB_ERR_RUNTIME, [&] { plan->engine->deviceStatus(device); });
}

float spnb_last_kernel_ms(const spnb_plan* plan) { return plan ? plan->engine->lastKernelMs() : 0.f; }

void spnb_plan_free(spnb_plan* plan) { delete plan; }

int spnb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

const char* spnb_last_error(void) { return g_lastError.c_str(); }
const char* spnb_version(void) { return "spnb 0.1 (sm_100a)"; }

}  // extern "C"
