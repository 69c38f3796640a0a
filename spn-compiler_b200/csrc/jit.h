// NVRTC front: CUDA C++ source -> sm_100a cubin.  Needs no GPU.
#pragma once
#include <string>
#include <vector>

namespace spnb {

struct JitResult {
  std::vector<char> cubin;
  std::string log;       // compiler log, includes the ptxas resource line (registers, spills)
  int registers = -1;    // parsed from the log, -1 if not found
  int spillBytes = -1;   // spill stores + loads in bytes, -1 if not found
};

// NVRTC version as major * 100 + minor (e.g. 1209).
int jitVersion();

// Throws std::runtime_error (message contains the compiler log) on failure.
JitResult jitCompile(const std::string& source, const std::string& name, int optLevel, int maxRegisters);

}  // namespace spnb
