// TEST INFRASTRUCTURE ONLY.  Compiles the reference profiler's own input
// generators (initMemrefF32 / initMemrefF16 / f32ToF16Bits, which live in
// fragment headers under backend/welder/compiler/solver/) behind a C ABI so
// golden vectors can be taken from the reference itself.  The headers are
// included from the reference tree where it lies; nothing is copied.  The
// fragments expect the includes, the MemrefDesc record and llvm::errs() that
// WelderProfiler.cpp provides before including them (WelderProfiler.cpp:1-56),
// so this shim provides the same surroundings: the standard headers, a record
// with the same fields, and a std::ostream stand-in for llvm::errs().
#include <cuda.h>

#include <algorithm>
#include <array>
#include <cctype>
#include <cerrno>
#include <charconv>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <limits>
#include <optional>
#include <sstream>
#include <string>
#include <string_view>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include <unistd.h>

namespace llvm {
inline std::ostream &errs() { return std::cerr; }
inline std::ostream &outs() { return std::cout; }
} // namespace llvm

namespace {
// Field-for-field the three records WelderProfiler.cpp:31-52 declares before
// it includes the fragments.
struct LaunchArg {
  std::string value;
  std::string type;
};
struct LaunchSpec {
  std::string binaryName;
  std::string entryName;
  std::array<std::string, 3> gridTokens;
  std::array<std::string, 3> blockTokens;
  std::vector<LaunchArg> args;
};
struct MemrefDesc {
  int rank = 0;
  std::string baseSym;
  std::string alignedSym;
  int64_t offset = 0;
  std::array<int64_t, 2> sizes = {0, 0};
  std::array<int64_t, 2> strides = {0, 0};
  int64_t bytes = 0;
};
#include "WelderProfilerParsing.h"
#include "WelderProfilerEval.h"
#include "WelderProfilerRuntime.h"
} // namespace

static MemrefDesc dense2d(int64_t rows, int64_t cols, int elemBytes) {
  MemrefDesc d;
  d.rank = 2;
  d.sizes = {rows, cols};
  d.strides = {cols, 1};
  d.bytes = rows * cols * elemBytes;
  return d;
}

extern "C" {
// mode: "zero" | "linear" | "random"
void ref_init_f32(float *buf, int64_t rows, int64_t cols, const char *mode, uint64_t seed) {
  initMemrefF32(dense2d(rows, cols, 4), buf, mode, seed);
}
void ref_init_f16(uint16_t *buf, int64_t rows, int64_t cols, const char *mode, uint64_t seed) {
  initMemrefF16(dense2d(rows, cols, 2), buf, mode, seed);
}
uint16_t ref_f32_to_f16_bits(float x) { return f32ToF16Bits(x); }
}
