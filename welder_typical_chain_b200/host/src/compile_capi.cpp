// libwelder-compile-capi.so: welder_compile_typical_chain_to_nvvm (C ABI) and
// welderCompilerMain (C++ linkage, callable repeatedly in one process).  Contract in
// include/welder_compile_capi.h.
#include "../../../include/welder_compile_capi.h"

#include "wtc_host.h"

#include <algorithm>
#include <cstring>
#include <filesystem>
#include <iostream>
#include <string>
#include <vector>

namespace {
void setError(char *buf, size_t n, const std::string &msg) {
  if (!buf || n == 0) return;
  const size_t k = std::min(n - 1, msg.size());
  std::memcpy(buf, msg.data(), k);
  buf[k] = '\0';
}
} // namespace

// argv as the reference's compile session assembles it (driver/WelderCompileSession.cpp:167-205):
// positional input, --force-tile-m/-n/-k v, --thread-tile-m/-n v, --max-connect-level v, the
// fused / baseline flag group, --output <03 path>.  Every other flag is accepted and ignored.
// With --emit-all-stages the 04 / 04c / 05 files and compile.log are written beside --output.
int welderCompilerMain(int argc, char **argv) {
  wtc::transform::CompileRequest req;
  std::string output;
  bool fusedSeen = false, allStages = false;
  try {
    for (int i = 1; i < argc; ++i) {
      const std::string a = argv[i];
      auto val = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
      if (a == "--force-tile-m") req.tileM = std::stoll(val());
      else if (a == "--force-tile-n") req.tileN = std::stoll(val());
      else if (a == "--force-tile-k") req.tileK = std::stoll(val());
      else if (a == "--thread-tile-m") req.threadTileM = std::stoll(val());
      else if (a == "--thread-tile-n") req.threadTileN = std::stoll(val());
      else if (a == "--max-connect-level") req.maxConnectLevel = std::stoll(val());
      else if (a == "--output" || a == "-o") output = val();
      else if (a == "--emit-all-stages") allStages = true;
      else if (a == "--verbose") req.verbose = true;
      else if (a == "--reduction-chain-split-broadcast-edges=false" || a == "--enable-matmul-softmax-shared-reuse-fusion") { req.fused = true; fusedSeen = true; }
      else if (a == "--reduction-chain-split-broadcast-edges=true") { req.fused = false; fusedSeen = true; }
      else if (a.rfind("--", 0) == 0) continue;
      else if (req.inputMlirPath.empty()) req.inputMlirPath = a;
    }
  } catch (const std::exception &) {
    std::cerr << "error: bad numeric flag value\n";
    return 2;
  }
  if (!fusedSeen) req.fused = req.maxConnectLevel > 0;
  if (req.inputMlirPath.empty()) { std::cerr << "error: no input MLIR given\n"; return 2; }
  if (output.empty()) { std::cerr << "error: --output is required\n"; return 2; }
  std::string error;
  int rc;
  if (allStages) {
    req.outDir = std::filesystem::path(output).parent_path().string();
    if (req.outDir.empty()) req.outDir = ".";
    rc = wtc::transform::compileChainToPlan(req, error);
  } else {
    rc = wtc::transform::emitPostbufferizeStage(req, output, error);
  }
  if (rc != 0) std::cerr << "error: " << error << "\n";
  return rc;
}

extern "C" int welder_compile_typical_chain_to_nvvm(const char *input_mlir_path, const char *out_dir,
                                                    const char * /*workgroup_pass_plugin_path*/,
                                                    const char * /*welder_compiler_bin_path*/, int64_t tile_m, int64_t tile_n,
                                                    int64_t tile_k, int64_t thread_tile_m, int64_t thread_tile_n,
                                                    int64_t max_connect_level, int fused, int verbose, char *error_buffer,
                                                    size_t error_buffer_size) {
  setError(error_buffer, error_buffer_size, "");
  if (!input_mlir_path || !*input_mlir_path) { setError(error_buffer, error_buffer_size, "input_mlir_path is empty"); return 1; }
  if (!out_dir || !*out_dir) { setError(error_buffer, error_buffer_size, "out_dir is empty"); return 1; }
  if (tile_m <= 0 || tile_n <= 0 || tile_k <= 0 || thread_tile_m <= 0 || thread_tile_n <= 0) {
    setError(error_buffer, error_buffer_size, "invalid tile sizes");
    return 1;
  }
  // Stage 1 goes through welderCompilerMain with the same argv the reference assembles, so the
  // in-process entry is exercised on every API compile; the later stages follow here.
  const std::string stage03 = (std::filesystem::path(out_dir) / "03.after_postbufferize.mlir").string();
  std::error_code ec;
  std::filesystem::create_directories(out_dir, ec);
  if (ec) { setError(error_buffer, error_buffer_size, std::string("failed to create out_dir: ") + out_dir); return 2; }
  std::vector<std::string> args = {"welder-compiler", input_mlir_path, "--enable-generic-problem", "--enable-tile-propagation",
                                   "--enable-cut-edges", "--enable-two-level-schedule", "--require-perfect-tiling=false",
                                   "--force-tile-m", std::to_string(tile_m), "--force-tile-n", std::to_string(tile_n),
                                   "--force-tile-k", std::to_string(tile_k), "--enable-register-level-schedule",
                                   "--thread-tile-m", std::to_string(thread_tile_m), "--thread-tile-n", std::to_string(thread_tile_n),
                                   "--max-connect-level", std::to_string(max_connect_level)};
  if (fused) {
    args.insert(args.end(), {"--reduction-chain-split-broadcast-edges=false", "--enable-row-reduction-chain-reuse-fusion",
                             "--enable-row-reduction-input-promotion", "--enable-matmul-softmax-shared-reuse-fusion"});
  } else {
    args.push_back("--reduction-chain-split-broadcast-edges=true");
  }
  args.push_back("--output");
  args.push_back(stage03);
  std::vector<char *> argv;
  for (std::string &s : args) argv.push_back(const_cast<char *>(s.c_str()));
  if (welderCompilerMain(static_cast<int>(argv.size()), argv.data()) != 0) {
    setError(error_buffer, error_buffer_size, "welder-compiler in-process failed (chain not recognised?)");
    return 2;
  }
  wtc::transform::CompileRequest req;
  req.inputMlirPath = input_mlir_path;
  req.outDir = out_dir;
  req.tileM = tile_m; req.tileN = tile_n; req.tileK = tile_k;
  req.threadTileM = thread_tile_m; req.threadTileN = thread_tile_n;
  req.maxConnectLevel = max_connect_level;
  req.fused = fused != 0;
  req.verbose = verbose != 0;
  std::string error;
  if (wtc::transform::compileChainToPlan(req, error) != 0) { setError(error_buffer, error_buffer_size, error); return 2; }
  return 0;
}
