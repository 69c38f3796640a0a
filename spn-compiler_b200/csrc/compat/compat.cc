#include <sys/stat.h>

#include <stdexcept>
#include <vector>

#include "../../../include/spnb.h"
#include "spnc-runtime.h"
#include "spnc.h"

namespace spnc {

Kernel spn_compiler::compileQuery(const std::string& inputFile, const options_t& options) {
  std::vector<const char*> keys, vals;
  for (auto& kv : options) {
    keys.push_back(kv.first.c_str());
    vals.push_back(kv.second.c_str());
  }
  char path[4096];
  spnb_kernel_info info;
  int rc = spnb_compile(inputFile.c_str(), keys.data(), vals.data(), (int)keys.size(), nullptr, path, sizeof path, &info);
  if (rc != SPNB_OK) throw std::runtime_error(std::string("COMPILATION ERROR: ") + spnb_last_error());
  return Kernel(path, info.kernel_name, info.query_type, info.target, info.batch_size, info.num_features,
                info.bytes_per_feature, info.num_results, info.bytes_per_result, info.dtype);
}

bool spn_compiler::isTargetSupported(const std::string& target) {
  if (target == "CUDA") return spnb_device_count() > 0;
  return false;  // the CPU code generator of the reference is not part of this engine
}

bool spn_compiler::isFeatureSupported(const std::string& feature) {
  // the reference answers CPU vectorisation questions here (compiler/src/Driver.cpp:61-82); none apply
  (void)feature;
  return false;
}

std::string spn_compiler::getHostArchitecture() {
#if defined(__x86_64__)
  return "x86_64";
#elif defined(__aarch64__)
  return "aarch64";
#else
  return "unknown";
#endif
}

}  // namespace spnc

namespace spnc_rt {

struct spn_runtime::Entry {
  spnb_plan* plan = nullptr;
  ~Entry() {
    if (plan) spnb_plan_free(plan);
  }
};

spn_runtime::~spn_runtime() = default;

spn_runtime& spn_runtime::instance() {
  static spn_runtime* rt = new spn_runtime();  // never destroyed: CUDA may already be gone at exit
  return *rt;
}

static std::string cacheKey(const spnc::Kernel& k) {
  struct stat st {};
  std::string key = k.fileName() + "|" + k.kernelName();
  if (stat(k.fileName().c_str(), &st) == 0)
    key += "|" + std::to_string((long long)st.st_size) + "|" + std::to_string((long long)st.st_mtim.tv_sec) + "." +
           std::to_string((long long)st.st_mtim.tv_nsec);
  return key;
}

void spn_runtime::execute(const spnc::Kernel& kernel, size_t num_elements, void* inputs, void* outputs) {
  if (kernel.target() != spnc::KernelTarget::CUDA)
    throw std::runtime_error("RUNTIME ERROR: this runtime only executes kernels compiled for the CUDA target");
  spnb_plan* plan = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu_);
    std::string key = cacheKey(kernel);
    auto it = cache_.find(key);
    if (it == cache_.end()) {
      std::unique_ptr<Entry> e(new Entry());
      if (spnb_plan_load(kernel.fileName().c_str(), &e->plan) != SPNB_OK)
        throw std::runtime_error(std::string("RUNTIME ERROR: ") + spnb_last_error());
      it = cache_.emplace(key, std::move(e)).first;
    }
    plan = it->second->plan;
  }
  if (spnb_execute_host(plan, num_elements, inputs, outputs) != SPNB_OK)
    throw std::runtime_error(std::string("RUNTIME ERROR: ") + spnb_last_error());
}

void spn_runtime::release(const spnc::Kernel& kernel) {
  std::lock_guard<std::mutex> lock(mu_);
  std::string prefix = kernel.fileName() + "|" + kernel.kernelName();
  for (auto it = cache_.begin(); it != cache_.end();) {
    if (it->first.compare(0, prefix.size(), prefix) == 0) it = cache_.erase(it);
    else ++it;
  }
}

}  // namespace spnc_rt
