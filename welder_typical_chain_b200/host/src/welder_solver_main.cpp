// welder-solver: CLI over the tile chooser, for the process_chain backend mode.  Accepts the
// flag set the front-end assembles (compiler/scheduler/SearchCommon.cpp:9-27 in the reference);
// flags that steer the reference's generic solver are accepted and ignored.  --enable-profiling
// measures the best-ranked implemented tiles on the device (solver/WelderSolver.cpp:202-213,479-513).
#include "wtc_host.h"

#include <iostream>
#include <string>

int main(int argc, char **argv) {
  std::string input, bestSummary, candidates;
  int64_t level = 1;
  wtc::scheduler::ProfileOptions prof;
  // value of `--flag v` or `--flag=v`
  auto valueOf = [&](const std::string &a, const char *flag, int &i, std::string &out) {
    const std::string f = flag;
    if (a == f && i + 1 < argc) { out = argv[++i]; return true; }
    if (a.rfind(f + "=", 0) == 0) { out = a.substr(f.size() + 1); return true; }
    return false;
  };
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    std::string v;
    if (a == "--enable-profiling" || a == "--enable-profiling=true") { prof.enable = true; continue; }
    if (a == "--profile-verbose") { prof.verbose = true; continue; }
    if (valueOf(a, "--schedule-topk", i, v)) { prof.topK = std::stoll(v); continue; }
    if (valueOf(a, "--profile-warmup", i, v)) { prof.warmup = std::stoi(v); continue; }
    if (valueOf(a, "--profile-iters", i, v)) { prof.iters = std::stoi(v); continue; }
    if (valueOf(a, "--profile-cache", i, v)) { prof.cachePath = v; continue; }
    if (valueOf(a, "--profile-profiler-bin", i, v)) { prof.profilerBin = v; continue; }
    if (a == "--dump-best-summary-json" && i + 1 < argc) bestSummary = argv[++i];
    else if (a == "--dump-candidates-tsv" && i + 1 < argc) candidates = argv[++i];
    else if (a == "--max-connect-level" && i + 1 < argc) level = std::stoll(argv[++i]);
    else if (a.rfind("--", 0) == 0) continue;
    else if (input.empty()) input = a;
  }
  if (input.empty()) { std::cerr << "usage: welder-solver <chain.mlir> [--max-connect-level n] [--dump-best-summary-json p] [--dump-candidates-tsv p]\n"
                            "       [--enable-profiling [--schedule-topk k] [--profile-warmup n] [--profile-iters n] [--profile-cache file] [--profile-profiler-bin path] [--profile-verbose]]\n"; return 2; }
  wtc::scheduler::SearchResult best;
  std::string error;
  const int rc = wtc::scheduler::solveTypicalChain(input, bestSummary, candidates, level, best, error, prof.enable ? &prof : nullptr);
  if (rc != 0) { std::cerr << "error: " << error << "\n"; return rc; }
  std::cout << "best: tileM=" << best.tileM << " tileN=" << best.tileN << " tileK=" << best.tileK << " threadTileM=" << best.threadTileM
            << " threadTileN=" << best.threadTileN << "\n";
  return 0;
}
