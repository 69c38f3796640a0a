#include "jit.h"

#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace spnb {

JitResult jitCompile(const std::string& source, const std::string& name, int optLevel, int maxRegisters) {
  nvrtcProgram prog;
  if (nvrtcCreateProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
    throw std::runtime_error("nvrtcCreateProgram failed");
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "--ftz=true",
                                   "--fmad=true", "--prec-div=true", "--prec-sqrt=true",
                                   "--ptxas-options=-v"};
  if (optLevel >= 0 && optLevel < 3) opts.push_back("--ptxas-options=-O" + std::to_string(optLevel));
  if (maxRegisters > 0) opts.push_back("--maxrregcount=" + std::to_string(maxRegisters));
  std::vector<const char*> copts;
  for (auto& s : opts) copts.push_back(s.c_str());
  nvrtcResult rc = nvrtcCompileProgram(prog, (int)copts.size(), copts.data());
  JitResult res;
  size_t logSize = 0;
  nvrtcGetProgramLogSize(prog, &logSize);
  if (logSize > 1) {
    res.log.resize(logSize);
    nvrtcGetProgramLog(prog, &res.log[0]);
  }
  if (rc != NVRTC_SUCCESS) {
    nvrtcDestroyProgram(&prog);
    throw std::runtime_error(std::string("NVRTC compilation failed: ") + nvrtcGetErrorString(rc) + "\n" + res.log);
  }
  size_t sz = 0;
  if (nvrtcGetCUBINSize(prog, &sz) != NVRTC_SUCCESS || sz == 0) {
    nvrtcDestroyProgram(&prog);
    throw std::runtime_error("NVRTC produced no cubin");
  }
  res.cubin.resize(sz);
  nvrtcGetCUBIN(prog, res.cubin.data());
  nvrtcDestroyProgram(&prog);
  // "Used 64 registers", "128 bytes spill stores, 132 bytes spill loads"
  size_t pos = res.log.find("Used ");
  if (pos != std::string::npos) res.registers = std::atoi(res.log.c_str() + pos + 5);
  pos = res.log.find(" bytes spill stores");
  if (pos != std::string::npos) {
    size_t b = res.log.rfind(' ', pos - 1);
    size_t nl = res.log.rfind('\n', pos);
    if (b == std::string::npos || (nl != std::string::npos && b < nl)) b = nl;
    int st = std::atoi(res.log.c_str() + (b == std::string::npos ? 0 : b + 1));
    size_t lp = res.log.find(" bytes spill loads", pos);
    int ld = 0;
    if (lp != std::string::npos) {
      size_t c = res.log.rfind(' ', lp - 1);
      ld = std::atoi(res.log.c_str() + c + 1);
    }
    res.spillBytes = st + ld;
  }
  return res;
}

}  // namespace spnb
