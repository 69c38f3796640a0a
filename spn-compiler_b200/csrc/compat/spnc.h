// spnc::spn_compiler -- compile an xspn query into a Kernel.
// Same static interface as the reference's compiler/include/spnc.h:18-48; implemented on the C ABI
// (spnb_compile).  Errors surface as std::runtime_error like the reference's SPNC_FATAL_ERROR
// (compiler/src/util/Logging.h:17-19).
#pragma once
#include <map>
#include <string>

#include "Kernel.h"

namespace spnc {

using options_t = std::map<std::string, std::string>;

class spn_compiler {
 public:
  static Kernel compileQuery(const std::string& inputFile, const options_t& options);
  static bool isTargetSupported(const std::string& target);
  static bool isFeatureSupported(const std::string& feature);
  static std::string getHostArchitecture();
};

}  // namespace spnc
