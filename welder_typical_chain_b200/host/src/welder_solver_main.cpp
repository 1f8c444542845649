// welder-solver: CLI over the tile chooser, for the process_chain backend mode.  Accepts the
// flag set the front-end assembles (compiler/scheduler/SearchCommon.cpp:9-27 in the reference);
// flags that steer the reference's generic solver are accepted and ignored.
#include "wtc_host.h"

#include <iostream>
#include <string>

int main(int argc, char **argv) {
  std::string input, bestSummary, candidates;
  int64_t level = 1;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--dump-best-summary-json" && i + 1 < argc) bestSummary = argv[++i];
    else if (a == "--dump-candidates-tsv" && i + 1 < argc) candidates = argv[++i];
    else if (a == "--max-connect-level" && i + 1 < argc) level = std::stoll(argv[++i]);
    else if (a.rfind("--", 0) == 0) continue;
    else if (input.empty()) input = a;
  }
  if (input.empty()) { std::cerr << "usage: welder-solver <chain.mlir> [--max-connect-level n] [--dump-best-summary-json p] [--dump-candidates-tsv p]\n"; return 2; }
  wtc::scheduler::SearchResult best;
  std::string error;
  const int rc = wtc::scheduler::solveTypicalChain(input, bestSummary, candidates, level, best, error);
  if (rc != 0) { std::cerr << "error: " << error << "\n"; return rc; }
  std::cout << "best: tileM=" << best.tileM << " tileN=" << best.tileN << " tileK=" << best.tileK << " threadTileM=" << best.threadTileM
            << " threadTileN=" << best.threadTileN << "\n";
  return 0;
}
