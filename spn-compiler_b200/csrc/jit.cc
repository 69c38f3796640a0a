#include "jit.h"

#include <dlfcn.h>
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace spnb {

namespace {

// NVRTC is loaded explicitly, by path, into its own namespace: a host process may already hold another
// NVRTC of the same soname (PyTorch bundles one), and which one the dynamic linker would hand out
// decides which PTX the JIT understands.  Order: $SPNB_NVRTC, the toolkit the library was built
// against, then the default search path.
struct Nvrtc {
  decltype(&nvrtcCreateProgram) createProgram = nullptr;
  decltype(&nvrtcCompileProgram) compileProgram = nullptr;
  decltype(&nvrtcGetProgramLogSize) getProgramLogSize = nullptr;
  decltype(&nvrtcGetProgramLog) getProgramLog = nullptr;
  decltype(&nvrtcGetCUBINSize) getCUBINSize = nullptr;
  decltype(&nvrtcGetCUBIN) getCUBIN = nullptr;
  decltype(&nvrtcDestroyProgram) destroyProgram = nullptr;
  decltype(&nvrtcGetErrorString) getErrorString = nullptr;
  decltype(&nvrtcVersion) version = nullptr;
  int major = 0, minor = 0;
  std::string path;

  static Nvrtc& get() {
    static Nvrtc n = load();
    return n;
  }
  static Nvrtc load() {
    std::vector<std::string> candidates;
    if (const char* e = std::getenv("SPNB_NVRTC")) candidates.push_back(e);
#ifdef SPNB_CUDA_HOME
    candidates.push_back(std::string(SPNB_CUDA_HOME) + "/lib64/libnvrtc.so.12");
    candidates.push_back(std::string(SPNB_CUDA_HOME) + "/lib64/libnvrtc.so");
#endif
    candidates.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
    candidates.push_back("libnvrtc.so.12");
    candidates.push_back("libnvrtc.so");
    std::string errors;
    for (auto& c : candidates) {
      void* h = dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (!h) {
        errors += std::string(" ") + (dlerror() ? dlerror() : c.c_str()) + ";";
        continue;
      }
      Nvrtc n;
      n.path = c;
      bool ok = true;
      auto sym = [&](const char* name, void** fn) {
        *fn = dlsym(h, name);
        if (!*fn) ok = false;
      };
      sym("nvrtcCreateProgram", (void**)&n.createProgram);
      sym("nvrtcCompileProgram", (void**)&n.compileProgram);
      sym("nvrtcGetProgramLogSize", (void**)&n.getProgramLogSize);
      sym("nvrtcGetProgramLog", (void**)&n.getProgramLog);
      sym("nvrtcGetCUBINSize", (void**)&n.getCUBINSize);
      sym("nvrtcGetCUBIN", (void**)&n.getCUBIN);
      sym("nvrtcDestroyProgram", (void**)&n.destroyProgram);
      sym("nvrtcGetErrorString", (void**)&n.getErrorString);
      sym("nvrtcVersion", (void**)&n.version);
      if (!ok) continue;
      n.version(&n.major, &n.minor);
      return n;
    }
    throw std::runtime_error("cannot load NVRTC (set SPNB_NVRTC to libnvrtc.so.12):" + errors);
  }
};

}  // namespace

int jitVersion() {
  Nvrtc& n = Nvrtc::get();
  return n.major * 100 + n.minor;
}

JitResult jitCompile(const std::string& source, const std::string& name, int optLevel, int maxRegisters) {
  Nvrtc& rt = Nvrtc::get();
  nvrtcProgram prog;
  if (rt.createProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
    throw std::runtime_error("nvrtcCreateProgram failed");
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "--ftz=true",
                                   "--fmad=true", "--prec-div=true", "--prec-sqrt=true",
                                   "--ptxas-options=-v"};
  if (optLevel >= 0 && optLevel < 3) opts.push_back("--ptxas-options=-O" + std::to_string(optLevel));
  if (maxRegisters > 0) opts.push_back("--maxrregcount=" + std::to_string(maxRegisters));
  std::vector<const char*> copts;
  for (auto& s : opts) copts.push_back(s.c_str());
  nvrtcResult rc = rt.compileProgram(prog, (int)copts.size(), copts.data());
  JitResult res;
  size_t logSize = 0;
  rt.getProgramLogSize(prog, &logSize);
  if (logSize > 1) {
    res.log.resize(logSize);
    rt.getProgramLog(prog, &res.log[0]);
  }
  if (rc != NVRTC_SUCCESS) {
    rt.destroyProgram(&prog);
    throw std::runtime_error(std::string("NVRTC compilation failed: ") + rt.getErrorString(rc) + "\n" + res.log);
  }
  size_t sz = 0;
  if (rt.getCUBINSize(prog, &sz) != NVRTC_SUCCESS || sz == 0) {
    rt.destroyProgram(&prog);
    throw std::runtime_error("NVRTC produced no cubin");
  }
  res.cubin.resize(sz);
  rt.getCUBIN(prog, res.cubin.data());
  rt.destroyProgram(&prog);
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
