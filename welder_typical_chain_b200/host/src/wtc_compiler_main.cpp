// wtc-compiler: the front-end CLI.  Flags, modes and exit codes (0 ok, 1 stage failure,
// 2 usage) follow the reference's compiler/main.cpp:11-117.  The command line is described by
// one table: flag spellings, whether a value follows, the help text and what the flag does.
#include "wtc_host.h"

#include <filesystem>
#include <functional>
#include <iostream>
#include <string>
#include <vector>

namespace {

using wtc::pipeline::RunMode;
using wtc::pipeline::RunOptions;

struct Cli {
  RunOptions run;
  int64_t repeat = 1;
  bool helpAsked = false;
  std::string error;     // set by a handler that rejects its value
};

struct Flag {
  std::vector<const char *> names;                              // first spelling is the documented one
  const char *valueName;                                        // nullptr: a switch
  const char *help;
  std::function<void(Cli &, const std::string &)> apply;
};

int64_t toInt(const std::string &v) { return std::stoll(v); }

const std::vector<Flag> &flagTable() {
  static const std::vector<Flag> table = {
      {{"--input"}, "mlir-file", "Chain to compile (required)", [](Cli &c, const std::string &v) { c.run.inputPath = v; }},
      {{"--output-dir", "--out-dir"}, "dir", "Output root dir (default /tmp/wtc_out)", [](Cli &c, const std::string &v) { c.run.outputDir = v; }},
      {{"--backend-root", "--legacy-root"}, "dir", "Backend root holding compiler/build/{welder-*,libwelder-*-capi.so}",
       [](Cli &c, const std::string &v) { c.run.backendRoot = v; }},
      {{"--backend-mode"}, "mode", "shell|process_chain|subprocess_pipeline|inprocess|api (default process_chain)",
       [](Cli &c, const std::string &v) {
         std::string diag;
         if (!wtc::backend::parseBackendMode(v, c.run.backendMode, diag)) c.error = diag;
       }},
      {{"--pure-api-full"}, nullptr, "Run search(api) and compile(api) in one process in full mode", [](Cli &c, const std::string &) { c.run.pureApiFull = true; }},
      {{"--search-only"}, nullptr, "Tile search only; writes search/best.json", [](Cli &c, const std::string &) { c.run.mode = RunMode::SearchOnly; }},
      {{"--compile-only"}, nullptr, "Compile; searches only when no tiles are given", [](Cli &c, const std::string &) { c.run.mode = RunMode::CompileOnly; }},
      {{"--best-json"}, "path", "Tile result to honour (tileM/N/K, threadTileM/N)", [](Cli &c, const std::string &v) { c.run.bestJsonPath = v; }},
      {{"--tile-m"}, "n", "Override tileM", [](Cli &c, const std::string &v) { c.run.tileM = toInt(v); }},
      {{"--tile-n"}, "n", "Override tileN", [](Cli &c, const std::string &v) { c.run.tileN = toInt(v); }},
      {{"--tile-k"}, "n", "Override tileK", [](Cli &c, const std::string &v) { c.run.tileK = toInt(v); }},
      {{"--thread-tile-m"}, "n", "Override threadTileM", [](Cli &c, const std::string &v) { c.run.threadTileM = toInt(v); }},
      {{"--thread-tile-n"}, "n", "Override threadTileN", [](Cli &c, const std::string &v) { c.run.threadTileN = toInt(v); }},
      {{"--max-connect-level"}, "n", "Connect level (0 = cut every edge)", [](Cli &c, const std::string &v) { c.run.maxConnectLevel = toInt(v); }},
      {{"--no-search"}, nullptr, "Never search; use --best-json, overrides or built-in defaults", [](Cli &c, const std::string &) { c.run.enableSearch = false; }},
      {{"--repeat"}, "n", "Repeat in one process into iter_<i>/ sub-directories", [](Cli &c, const std::string &v) { c.repeat = toInt(v); }},
      {{"--baseline"}, nullptr, "Compile the unfused variant (connect level forced to 0)",
       [](Cli &c, const std::string &) { c.run.fused = false; if (c.run.maxConnectLevel > 0) c.run.maxConnectLevel = 0; }},
      {{"--fused"}, nullptr, "Compile the fused variant (default)", [](Cli &c, const std::string &) { c.run.fused = true; }},
      {{"--verbose"}, nullptr, "Verbose logs", [](Cli &c, const std::string &) { c.run.verbose = true; }},
      {{"--help", "-h"}, nullptr, "This text", [](Cli &c, const std::string &) { c.helpAsked = true; }},
  };
  return table;
}

void printHelp() {
  std::cout << "Usage: wtc-compiler --input <mlir-file> [options]\nOptions:\n";
  for (const Flag &f : flagTable()) {
    std::string left = "  ";
    for (size_t i = 0; i < f.names.size(); ++i) left += std::string(i ? " | " : "") + f.names[i];
    if (f.valueName) left += std::string(" <") + f.valueName + ">";
    if (left.size() < 34) left.resize(34, ' ');
    std::cout << left << " " << f.help << "\n";
  }
}

const Flag *findFlag(const std::string &arg) {
  for (const Flag &f : flagTable())
    for (const char *n : f.names)
      if (arg == n) return &f;
  return nullptr;
}

} // namespace

int main(int argc, char **argv) {
  Cli cli;
  for (int i = 1; i < argc; ++i) {
    const std::string arg = argv[i];
    const Flag *flag = findFlag(arg);
    // a flag that takes a value but stands last is reported like an unknown one
    if (!flag || (flag->valueName && i + 1 >= argc)) { std::cerr << "Unknown argument: " << arg << "\n"; return 2; }
    try {
      flag->apply(cli, flag->valueName ? std::string(argv[++i]) : std::string());
    } catch (const std::exception &) {
      std::cerr << "error: bad numeric value for " << arg << "\n";
      return 2;
    }
    if (!cli.error.empty()) { std::cerr << "error: " << cli.error << "\n"; return 2; }
    if (cli.helpAsked) { printHelp(); return 0; }
  }
  if (cli.run.inputPath.empty()) { std::cerr << "error: --input is required\n"; return 2; }
  if (cli.repeat <= 0) { std::cerr << "error: --repeat must be >= 1\n"; return 2; }
  if (cli.repeat == 1) return wtc::pipeline::runTypicalChainPipeline(cli.run);
  for (int64_t i = 0; i < cli.repeat; ++i) {
    RunOptions once = cli.run;
    once.outputDir = (std::filesystem::path(cli.run.outputDir) / ("iter_" + std::to_string(i))).string();
    if (cli.run.verbose) std::cout << "[wtc] repeat " << (i + 1) << "/" << cli.repeat << ", output-dir=" << once.outputDir << "\n";
    const int rc = wtc::pipeline::runTypicalChainPipeline(once);
    if (rc != 0) { std::cerr << "error: repeat iteration failed at i=" << i << ", rc=" << rc << "\n"; return rc; }
  }
  return 0;
}
