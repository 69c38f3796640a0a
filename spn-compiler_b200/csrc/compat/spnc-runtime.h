// spnc_rt::spn_runtime -- execute a compiled Kernel on a batch held in host memory.
// Same interface as the reference's runtime/include/spnc-runtime.h:24-55.  Unlike the reference
// (runtime/src/runtime.cpp:33-49) the cache copies what it needs from the Kernel, is keyed by the plan
// file's path, size and modification time, and is guarded by a mutex.
#pragma once
#include <cstddef>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "Kernel.h"

struct spnb_plan;

namespace spnc_rt {

class spn_runtime {
 public:
  static spn_runtime& instance();
  // inputs: num_elements x numFeatures x bytesPerFeature bytes, row-major; outputs: num_elements x
  // numResults x bytesPerResult bytes; both owned by the caller.  Returns once outputs are written.
  void execute(const spnc::Kernel& kernel, size_t num_elements, void* inputs, void* outputs);
  // drops the cached plan of a kernel (e.g. before its file is deleted and the path reused)
  void release(const spnc::Kernel& kernel);

  spn_runtime(const spn_runtime&) = delete;
  spn_runtime& operator=(const spn_runtime&) = delete;

 private:
  spn_runtime() = default;
  ~spn_runtime();
  struct Entry;
  std::mutex mu_;
  std::unordered_map<std::string, std::unique_ptr<Entry>> cache_;
};

}  // namespace spnc_rt
