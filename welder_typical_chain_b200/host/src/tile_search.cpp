// Tile contract (best.json) and the B200 tile chooser.
//
// The reference searches a generic tile graph on a 48 KiB-smem / 80-SM arch model and
// ranks candidates by global-memory traffic x waves
// (backend/welder/compiler/solver/WelderSolverGraphAnalysisAndFootprintInfer.h:598-921,
// score at :818-821).  Here the operator is fixed, so the chooser enumerates the tile
// shapes that are legal for tcgen05 on sm_100a (M 128, N <= 256 per MMA, K a multiple of
// the 128-byte swizzle atom), filters them by shared-memory and tensor-memory footprint,
// and ranks them by the same traffic x waves product, computed on L2->SM operand bytes.
// The artifacts keep the reference's schema (solver/WelderSolverCAPI.cpp:40-100).
#include "wtc_host.h"

#include <algorithm>
#include <cmath>
#include <filesystem>
#include <fstream>
#include <regex>
#include <sstream>

namespace wtc::scheduler {
namespace {

bool extractInt64(const std::string &text, const char *key, int64_t &value) {
  const std::regex re(std::string("\"") + key + "\"\\s*:\\s*(-?[0-9]+)");
  std::smatch m;
  if (!std::regex_search(text, m, re) || m.size() < 2) return false;
  value = std::stoll(m[1].str());
  return true;
}

int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

} // namespace

// First occurrence of each key wins, so the flat best.json and the nested
// best_summary.json both load (compiler/scheduler/Search.cpp:35-60).
bool loadBestFromJson(const std::string &jsonPath, SearchResult &result, std::string &diagnostic) {
  if (jsonPath.empty()) { diagnostic = "json path is empty"; return false; }
  const std::string json = readAll(jsonPath);
  if (json.empty()) { diagnostic = "failed to read json: " + jsonPath; return false; }
  SearchResult parsed;
  if (!extractInt64(json, "tileM", parsed.tileM) || !extractInt64(json, "tileN", parsed.tileN) ||
      !extractInt64(json, "tileK", parsed.tileK) || !extractInt64(json, "threadTileM", parsed.threadTileM) ||
      !extractInt64(json, "threadTileN", parsed.threadTileN)) {
    diagnostic = "failed to parse tile fields from " + jsonPath;
    return false;
  }
  result = parsed;
  diagnostic.clear();
  return true;
}

bool writeBestToJson(const SearchResult &r, const std::string &jsonPath, std::string &diagnostic) {
  if (jsonPath.empty()) { diagnostic = "json path is empty"; return false; }
  std::ostringstream o;
  o << "{\n  \"tileM\": " << r.tileM << ",\n  \"tileN\": " << r.tileN << ",\n  \"tileK\": " << r.tileK
    << ",\n  \"threadTileM\": " << r.threadTileM << ",\n  \"threadTileN\": " << r.threadTileN << "\n}\n";
  if (!writeAll(jsonPath, o.str())) { diagnostic = "failed to open json for write: " + jsonPath; return false; }
  diagnostic.clear();
  return true;
}

std::vector<Candidate> enumerateCandidates(const ir::ChainSpec &spec, const ArchModel &arch, int64_t maxConnectLevel) {
  std::vector<Candidate> out;
  const bool f16 = spec.inType == "f16";
  const double eb = f16 ? 2.0 : 4.0;
  const double ob = spec.outType == "f16" ? 2.0 : 4.0;
  const double flops = 2.0 * spec.batch * spec.M * spec.N * spec.K;
  const bool fused = maxConnectLevel > 0;
  for (int64_t tm : {64, 128}) {
    for (int64_t tn : {64, 128, 256}) {
      for (int64_t tk : {32, 64, 128}) {
        // ---- footprint filters
        const int64_t stageBytes = (tm * tk + tk * tn) * static_cast<int64_t>(eb);
        const int64_t outStage = tm * tn * 2 / 2;                 // f16 staging, half a tile in flight
        const int64_t fixed = outStage + 2 * 8 * tm * 8 + 4096;   // + row statistics exchange + barriers
        const int64_t stages = std::min<int64_t>(8, (arch.smemBytes - fixed) / stageBytes);
        if (stages < 2) continue;
        if (2 * tn > arch.tmemColumns) continue;                  // two accumulator buffers
        const int64_t clusterN = ceilDiv(spec.N, tn);
        const bool twoPass = clusterN > 8;                        // row does not fit one portable cluster
        // ---- traffic: every row block re-reads B, every column block re-reads A (from L2)
        const double rb = static_cast<double>(ceilDiv(spec.M, tm)), nb = static_cast<double>(ceilDiv(spec.N, tn));
        const double bytesA = spec.batch * rb * nb * tm * static_cast<double>(spec.K) * eb;
        const double bytesB = spec.batch * rb * nb * tn * static_cast<double>(spec.K) * eb;
        double bytesC = spec.batch * static_cast<double>(spec.M) * spec.N * ob;
        double bytesCut = 0.0;                                    // intermediates that cross global memory
        if (!fused) bytesCut = spec.batch * static_cast<double>(spec.M) * spec.N * 4.0 * 4.0;   // C32 and E, written + read
        else if (twoPass) bytesCut = 2.0 * bytesC;                // the rescale pass re-reads and re-writes the output
        const double ctas = spec.batch * rb * nb;
        const double waves = std::ceil(ctas / static_cast<double>(arch.numSM));
        Candidate c;
        c.tileM = tm; c.tileN = tn; c.tileK = tk;
        c.threadTileM = 1; c.threadTileN = std::max<int64_t>(1, tn / 2);   // one epilogue thread: one row x half the tile
        c.stages = static_cast<int>(stages);
        c.clusterN = twoPass ? 1 : static_cast<int>(clusterN);
        c.implemented = f16 && tm == 128 && (tn == 256 || tn == 128) && tk == 64;   // tile shapes the kernel library has
        c.bytesA = bytesA; c.bytesB = bytesB; c.bytesC = bytesC; c.bytesCut = bytesCut;
        c.score = (bytesA + bytesB + bytesC + bytesCut) * waves;
        // latency model: the slowest of tensor time (M=64 MMAs run at half rate), L2 operand feed,
        // HBM compulsory traffic and the MUFU-bound softmax epilogue (16 ex2/clk/SM), plus a fill term
        const double tensorUs = flops / (arch.tensorTflops * 1e6) * (tm == 64 ? 2.0 : 1.0) * (tn < 256 ? 1.15 : 1.0);
        const double l2Us = (bytesA + bytesB) / (arch.l2TBps * 1e6);
        const double compulsory = eb * (spec.batch * static_cast<double>(spec.M) * spec.K +
                                        (spec.bBatched ? spec.batch : 1) * static_cast<double>(spec.K) * spec.N);
        const double hbmUs = (compulsory + bytesC + bytesCut) / (arch.hbmTBps * 1e6);
        const double mufuUs = spec.batch * static_cast<double>(spec.M) * spec.N / (16.0 * arch.numSM * 1.9e3);
        const double occupancy = std::min(1.0, ctas / static_cast<double>(arch.numSM));
        c.estimatedLatencyUs = std::max({tensorUs / occupancy, l2Us, hbmUs, mufuUs / occupancy}) + 2.0;
        out.push_back(c);
      }
    }
  }
  std::stable_sort(out.begin(), out.end(), [](const Candidate &x, const Candidate &y) {
    if (x.implemented != y.implemented) return x.implemented;
    if (x.score != y.score) return x.score < y.score;
    return x.estimatedLatencyUs < y.estimatedLatencyUs;
  });
  return out;
}

bool writeBestSummaryJson(const ir::ChainSpec &spec, const ArchModel &arch, const std::vector<Candidate> &sorted,
                          const std::string &path, std::string &error) {
  if (sorted.empty()) { error = "empty candidate list"; return false; }
  const Candidate &b = sorted.front();
  std::ostringstream o;
  o.precision(9);
  o << "{\n"
    << "  \"problem\": {\"m\": " << spec.M << ", \"n\": " << spec.N << ", \"k\": " << spec.K << ", \"batch\": " << spec.batch << "},\n"
    << "  \"arch\": {\"smemBytes\": " << arch.smemBytes << ", \"numSM\": " << arch.numSM << ", \"warpSize\": " << arch.warpSize
    << ", \"elementBytes\": " << (spec.inType == "f16" ? 2 : 4) << ", \"tmemColumns\": " << arch.tmemColumns << ", \"chip\": \"sm_100a\"},\n"
    << "  \"best\": {\"tileM\": " << b.tileM << ", \"tileN\": " << b.tileN << ", \"tileK\": " << b.tileK
    << ", \"threadTileM\": " << b.threadTileM << ", \"threadTileN\": " << b.threadTileN << ", \"score\": " << b.score
    << ", \"estimatedLatency\": " << b.estimatedLatencyUs << ", \"profiledMs\": -1, \"bytesCut\": " << b.bytesCut
    << ", \"stages\": " << b.stages << ", \"clusterN\": " << b.clusterN << ", \"implemented\": " << (b.implemented ? "true" : "false") << "}\n"
    << "}\n";
  if (!writeAll(path, o.str())) { error = "failed to open best summary json: " + path; return false; }
  return true;
}

bool writeCandidatesTsv(const std::vector<Candidate> &sorted, const std::string &path, std::string &error) {
  std::ostringstream o;
  o.precision(9);
  o << "rank\ttileM\ttileN\ttileK\tthreadTileM\tthreadTileN\tscore\testimatedLatency\tprofiledMs\tbytesA\tbytesB\tbytesC\tbytesCut\n";
  for (size_t i = 0; i < sorted.size(); ++i) {
    const Candidate &c = sorted[i];
    o << i << "\t" << c.tileM << "\t" << c.tileN << "\t" << c.tileK << "\t" << c.threadTileM << "\t" << c.threadTileN << "\t" << c.score
      << "\t" << c.estimatedLatencyUs << "\t-1\t" << c.bytesA << "\t" << c.bytesB << "\t" << c.bytesC << "\t" << c.bytesCut << "\n";
  }
  if (!writeAll(path, o.str())) { error = "failed to open candidates tsv: " + path; return false; }
  return true;
}

// rc: 0 ok, 2 open/parse failure, 3 no candidates, 4 I/O failure (solver/WelderSolverCAPI.cpp:104-196)
int solveTypicalChain(const std::string &inputMlir, const std::string &bestSummaryJson, const std::string &candidatesTsv,
                      int64_t maxConnectLevel, SearchResult &best, std::string &error) {
  trace::Span span("search");
  ir::ChainSpec spec;
  if (!ir::parseChainFile(inputMlir, spec, error)) { span.fail(); return 2; }
  const ArchModel arch;
  const std::vector<Candidate> sorted = enumerateCandidates(spec, arch, maxConnectLevel);
  if (sorted.empty()) { error = "no legal tile candidate for this chain"; span.fail(); return 3; }
  if (!bestSummaryJson.empty() && !writeBestSummaryJson(spec, arch, sorted, bestSummaryJson, error)) { span.fail(); return 4; }
  if (!candidatesTsv.empty() && !writeCandidatesTsv(sorted, candidatesTsv, error)) { span.fail(); return 4; }
  const Candidate &b = sorted.front();
  best.tileM = b.tileM; best.tileN = b.tileN; best.tileK = b.tileK;
  best.threadTileM = b.threadTileM; best.threadTileN = b.threadTileN;
  error.clear();
  return 0;
}

} // namespace wtc::scheduler
