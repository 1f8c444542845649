// wtc-compiler: the front-end CLI.  Flags, modes and exit codes (0 ok, 1 stage failure,
// 2 usage) follow the reference's compiler/main.cpp:11-117.
#include "wtc_host.h"

#include <filesystem>
#include <iostream>
#include <string>

int main(int argc, char **argv) {
  wtc::pipeline::RunOptions options;
  int64_t repeat = 1;
  auto need = [&](int i) { return i + 1 < argc; };
  for (int i = 1; i < argc; ++i) {
    const std::string arg = argv[i];
    try {
      if (arg == "--input" && need(i)) options.inputPath = argv[++i];
      else if ((arg == "--output-dir" || arg == "--out-dir") && need(i)) options.outputDir = argv[++i];
      else if ((arg == "--backend-root" || arg == "--legacy-root") && need(i)) options.backendRoot = argv[++i];
      else if (arg == "--best-json" && need(i)) options.bestJsonPath = argv[++i];
      else if (arg == "--backend-mode" && need(i)) {
        std::string diag;
        if (!wtc::backend::parseBackendMode(argv[++i], options.backendMode, diag)) { std::cerr << "error: " << diag << "\n"; return 2; }
      } else if (arg == "--max-connect-level" && need(i)) options.maxConnectLevel = std::stoll(argv[++i]);
      else if (arg == "--tile-m" && need(i)) options.tileM = std::stoll(argv[++i]);
      else if (arg == "--tile-n" && need(i)) options.tileN = std::stoll(argv[++i]);
      else if (arg == "--tile-k" && need(i)) options.tileK = std::stoll(argv[++i]);
      else if (arg == "--thread-tile-m" && need(i)) options.threadTileM = std::stoll(argv[++i]);
      else if (arg == "--thread-tile-n" && need(i)) options.threadTileN = std::stoll(argv[++i]);
      else if (arg == "--no-search") options.enableSearch = false;
      else if (arg == "--pure-api-full") options.pureApiFull = true;
      else if (arg == "--repeat" && need(i)) repeat = std::stoll(argv[++i]);
      else if (arg == "--search-only") options.mode = wtc::pipeline::RunMode::SearchOnly;
      else if (arg == "--compile-only") options.mode = wtc::pipeline::RunMode::CompileOnly;
      else if (arg == "--baseline") { options.fused = false; if (options.maxConnectLevel > 0) options.maxConnectLevel = 0; }
      else if (arg == "--fused") options.fused = true;
      else if (arg == "--verbose") options.verbose = true;
      else if (arg == "--help" || arg == "-h") {
        std::cout << "Usage: wtc-compiler --input <mlir-file> [options]\n"
                     "Options:\n"
                     "  --output-dir <dir>       Output root dir (default /tmp/wtc_out); alias --out-dir\n"
                     "  --backend-root <dir>     Backend root holding compiler/build/{welder-*,libwelder-*-capi.so}; alias --legacy-root\n"
                     "  --backend-mode <mode>    shell|process_chain|subprocess_pipeline|inprocess|api (default process_chain)\n"
                     "  --pure-api-full          Run search(api) and compile(api) in one process in full mode\n"
                     "  --search-only            Tile search only; writes search/best.json\n"
                     "  --compile-only           Compile; searches only when no tiles are given\n"
                     "  --best-json <path>       Tile result to honour (tileM/N/K, threadTileM/N)\n"
                     "  --tile-m|-n|-k <n>       Override one tile size\n"
                     "  --thread-tile-m|-n <n>   Override one thread tile size\n"
                     "  --max-connect-level <n>  Connect level (0 = cut every edge)\n"
                     "  --no-search              Never search; use --best-json, overrides or built-in defaults\n"
                     "  --repeat <n>             Repeat in one process into iter_<i>/ sub-directories\n"
                     "  --baseline | --fused     Variant to compile (default --fused)\n"
                     "  --verbose                Verbose logs\n";
        return 0;
      } else { std::cerr << "Unknown argument: " << arg << "\n"; return 2; }
    } catch (const std::exception &) {
      std::cerr << "error: bad numeric value for " << arg << "\n";
      return 2;
    }
  }
  if (options.inputPath.empty()) { std::cerr << "error: --input is required\n"; return 2; }
  if (repeat <= 0) { std::cerr << "error: --repeat must be >= 1\n"; return 2; }
  if (repeat == 1) return wtc::pipeline::runTypicalChainPipeline(options);
  for (int64_t i = 0; i < repeat; ++i) {
    wtc::pipeline::RunOptions it = options;
    it.outputDir = (std::filesystem::path(options.outputDir) / ("iter_" + std::to_string(i))).string();
    if (options.verbose) std::cout << "[wtc] repeat " << (i + 1) << "/" << repeat << ", output-dir=" << it.outputDir << "\n";
    const int rc = wtc::pipeline::runTypicalChainPipeline(it);
    if (rc != 0) { std::cerr << "error: repeat iteration failed at i=" << i << ", rc=" << rc << "\n"; return rc; }
  }
  return 0;
}
