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

#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
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
        // tile shapes the kernel library has (the rule of tc_stage_depth_legal in csrc/fused_tc_kernel.cu):
        // 128 x {128,256} x 64 always; with f16 probabilities in the fused variant also 32-deep stages,
        // 128-deep stages (with 256 columns only in the two-pass schedule) and 64-row tiles (stages 32 or 64 deep)
        const bool wide = tn == 256 || tn == 128;
        const bool family = fused && spec.outType == "f16";
        c.implemented = f16 && wide &&
                        ((tm == 128 && tk == 64) ||
                         (family && tm == 128 && (tk == 32 || (tk == 128 && (tn == 128 || twoPass)))) ||
                         (family && tm == 64 && (tk == 32 || tk == 64)));
        c.bytesA = bytesA; c.bytesB = bytesB; c.bytesC = bytesC; c.bytesCut = bytesCut;
        c.score = (bytesA + bytesB + bytesC + bytesCut) * waves;
        // latency model: the slowest of tensor time (M=64 MMAs run at half rate), L2 operand feed,
        // HBM compulsory traffic and the MUFU-bound softmax epilogue (16 ex2/clk/SM), plus a fill term.
        // Tensor time counts rounds: a cluster of n CTAs is resident only kResident[n] times on the part.
        static const int kResident[9] = {0, 148, 72, 47, 35, 27, 22, 18, 15};
        const double parallel = twoPass ? std::min<double>(ctas, static_cast<double>(arch.numSM))
                                        : std::min<double>(ctas, static_cast<double>(kResident[clusterN]) * static_cast<double>(clusterN));
        const double rounds = std::ceil(ctas / std::max(1.0, parallel));
        const double perTileUs = 2.0 * tm * tn * static_cast<double>(spec.K) / (arch.tensorTflops / static_cast<double>(arch.numSM) * 1e6) *
                                 (tm == 64 ? 2.0 : 1.0) * (tn < 256 ? 1.15 : 1.0);
        const double tensorUs = perTileUs * rounds;
        const double l2Us = (bytesA + bytesB) / (arch.l2TBps * 1e6);
        const double compulsory = eb * (spec.batch * static_cast<double>(spec.M) * spec.K +
                                        (spec.bBatched ? spec.batch : 1) * static_cast<double>(spec.K) * spec.N);
        const double hbmUs = (compulsory + bytesC + bytesCut) / (arch.hbmTBps * 1e6);
        const double mufuUs = static_cast<double>(tm) * tn / (16.0 * 1.9e3) * rounds;
        c.estimatedLatencyUs = std::max({tensorUs, l2Us, hbmUs, mufuUs}) + 2.0;
        out.push_back(c);
      }
    }
  }
  std::stable_sort(out.begin(), out.end(), [](const Candidate &x, const Candidate &y) {
    if (x.implemented != y.implemented) return x.implemented;
    // among tiles that have kernels the latency model decides (it knows about idle SMs and
    // cluster residency); the rest keep the reference's traffic x waves order
    if (x.implemented && x.estimatedLatencyUs != y.estimatedLatencyUs) return x.estimatedLatencyUs < y.estimatedLatencyUs;
    // the model does not see the stage depth: the 64-deep kernels are the tuned ones (on-device
    // profiling of the candidates, when enabled, replaces this order with measured times)
    if (x.implemented && (x.tileK == 64) != (y.tileK == 64)) return x.tileK == 64;
    if (x.score != y.score) return x.score < y.score;
    return x.estimatedLatencyUs < y.estimatedLatencyUs;
  });
  return out;
}


// ---- on-device profiling of the top-k candidates ------------------------------------------

std::string buildProfileKey(const ir::ChainSpec &spec, const Candidate &c, int64_t maxConnectLevel) {
  std::ostringstream k;
  k << "wtc_b200_chain|batch=" << spec.batch << "|m=" << spec.M << "|n=" << spec.N << "|k=" << spec.K << "|bb=" << (spec.bBatched ? 1 : 0)
    << "|in=" << spec.inType << "|acc=" << spec.accType << "|out=" << spec.outType << "|scale=" << spec.scale
    << "|tile=" << c.tileM << "x" << c.tileN << "x" << c.tileK << "|level=" << maxConnectLevel
    // raised when the kernels behind a tile change enough to make old timings misleading
    << "|profile_key_rev=sm100a_relay_v2";
  return k.str();
}

namespace {

// directory that holds the module this code is linked into (the solver binary or C-API library)
std::string moduleDir() {
  Dl_info info;
  if (dladdr(reinterpret_cast<const void *>(&moduleDir), &info) && info.dli_fname) {
    std::error_code ec;
    const std::filesystem::path p = std::filesystem::canonical(info.dli_fname, ec);
    if (!ec) return p.parent_path().string();
  }
  return ".";
}

void loadProfileCache(const std::string &path, std::map<std::string, double> &cache) {
  if (path.empty()) return;
  std::ifstream in(path);
  std::string line;
  while (std::getline(in, line)) {
    const size_t tab = line.find('\t');
    if (line.empty() || tab == std::string::npos) continue;
    const double ms = std::strtod(line.c_str() + tab + 1, nullptr);
    if (ms > 0.0) cache[line.substr(0, tab)] = ms;   // later lines win
  }
}

void appendProfileCache(const std::string &path, const std::string &key, double ms) {
  if (path.empty()) return;
  std::ofstream out(path, std::ios::out | std::ios::app);
  if (out) out << key << "\t" << ms << "\n";
}

// runs `cmd`, returns its stdout; rc gets the exit status
std::string captureCommand(const std::string &cmd, int &rc) {
  std::string out;
  FILE *f = popen(cmd.c_str(), "r");
  if (!f) { rc = -1; return out; }
  char buf[512];
  while (fgets(buf, sizeof buf, f)) out += buf;
  const int st = pclose(f);
  rc = st == -1 ? -1 : (WIFEXITED(st) ? WEXITSTATUS(st) : 128);
  return out;
}

std::string quote(const std::string &s) {
  std::string q = "'";
  for (char ch : s) { if (ch == '\'') q += "'\\''"; else q += ch; }
  return q + "'";
}

} // namespace

int profileCandidates(const std::string &inputMlir, const ir::ChainSpec &spec, int64_t maxConnectLevel,
                      const ProfileOptions &opts, std::vector<Candidate> &sorted, std::string &log) {
  trace::Span span("profile");
  std::ostringstream lg;
  std::map<std::string, double> cache;
  loadProfileCache(opts.cachePath, cache);
  const std::string profiler = opts.profilerBin.empty() ? moduleDir() + "/welder-profiler" : opts.profilerBin;
  std::error_code ec;
  const std::filesystem::path tmpRoot = std::filesystem::temp_directory_path(ec) / ("wtc_profile_" + std::to_string(static_cast<long long>(getpid())));
  int measured = 0;
  int64_t taken = 0;
  for (size_t i = 0; i < sorted.size() && taken < opts.topK; ++i) {
    Candidate &c = sorted[i];
    if (!c.implemented) continue;          // no kernel behind this tile: nothing to run
    ++taken;
    const std::string key = buildProfileKey(spec, c, maxConnectLevel);
    const auto hit = cache.find(key);
    if (hit != cache.end()) {
      c.profiledMs = hit->second;
      ++measured;
      lg << "[wtc.profile] cache hit  tile " << c.tileM << "x" << c.tileN << "x" << c.tileK << " -> " << c.profiledMs << " ms\n";
      continue;
    }
    transform::CompileRequest req;
    req.inputMlirPath = inputMlir;
    req.outDir = (tmpRoot / ("cand_" + std::to_string(i))).string();
    req.tileM = c.tileM; req.tileN = c.tileN; req.tileK = c.tileK;
    req.threadTileM = c.threadTileM; req.threadTileN = c.threadTileN;
    req.maxConnectLevel = maxConnectLevel;
    req.fused = maxConnectLevel > 0;
    std::string err;
    if (transform::compileChainToPlan(req, err) != 0) {
      lg << "[wtc.profile] compile failed for tile " << c.tileM << "x" << c.tileN << "x" << c.tileK << ": " << err << "\n";
      continue;
    }
    const std::string cmd = quote(profiler) + " --warmup=" + std::to_string(opts.warmup) + " --iters=" + std::to_string(opts.iters) +
                            " --init=random " + quote(req.outDir + "/05.out.nvvm.runnable.mlir") + " 2>&1";
    int rc = 0;
    const std::string out = captureCommand(cmd, rc);
    std::smatch m;
    static const std::regex re("avg_ms=([-+0-9.eE]+)");
    if (rc == 0 && std::regex_search(out, m, re)) {
      const double ms = std::strtod(m[1].str().c_str(), nullptr);
      if (ms > 0.0) {
        c.profiledMs = ms;
        cache[key] = ms;
        appendProfileCache(opts.cachePath, key, ms);
        ++measured;
        lg << "[wtc.profile] measured   tile " << c.tileM << "x" << c.tileN << "x" << c.tileK << " -> " << ms << " ms\n";
        continue;
      }
    }
    lg << "[wtc.profile] run failed for tile " << c.tileM << "x" << c.tileN << "x" << c.tileK << " (rc " << rc << "): "
       << out.substr(0, 300) << "\n";
  }
  if (!opts.verbose) std::filesystem::remove_all(tmpRoot, ec);
  // measured candidates first, fastest first; the rest keep their model order
  std::stable_sort(sorted.begin(), sorted.end(), [](const Candidate &x, const Candidate &y) {
    const bool mx = x.profiledMs > 0.0, my = y.profiledMs > 0.0;
    if (mx != my) return mx;
    if (mx && my && x.profiledMs != y.profiledMs) return x.profiledMs < y.profiledMs;
    return false;
  });
  if (measured == 0) span.fail();
  log = lg.str();
  return measured;
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
    << ", \"estimatedLatency\": " << b.estimatedLatencyUs << ", \"profiledMs\": " << b.profiledMs << ", \"bytesCut\": " << b.bytesCut
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
      << "\t" << c.estimatedLatencyUs << "\t" << c.profiledMs << "\t" << c.bytesA << "\t" << c.bytesB << "\t" << c.bytesC << "\t" << c.bytesCut << "\n";
  }
  if (!writeAll(path, o.str())) { error = "failed to open candidates tsv: " + path; return false; }
  return true;
}

// rc: 0 ok, 2 open/parse failure, 3 no candidates, 4 I/O failure (solver/WelderSolverCAPI.cpp:104-196)
int solveTypicalChain(const std::string &inputMlir, const std::string &bestSummaryJson, const std::string &candidatesTsv,
                      int64_t maxConnectLevel, SearchResult &best, std::string &error, const ProfileOptions *profile) {
  trace::Span span("search");
  ir::ChainSpec spec;
  if (!ir::parseChainFile(inputMlir, spec, error)) { span.fail(); return 2; }
  const ArchModel arch;
  std::vector<Candidate> sorted = enumerateCandidates(spec, arch, maxConnectLevel);
  if (sorted.empty()) { error = "no legal tile candidate for this chain"; span.fail(); return 3; }
  // Profiling is asked for by the caller (welder-solver --enable-profiling) or, for callers
  // that go through the fixed C signature, by WTC_SOLVER_PROFILE=1 (+ _CACHE, _TOPK, _ITERS).
  ProfileOptions envProfile;
  if (!profile) {
    const char *e = std::getenv("WTC_SOLVER_PROFILE");
    if (e && e[0] == '1') {
      envProfile.enable = true;
      if (const char *v = std::getenv("WTC_SOLVER_PROFILE_CACHE")) envProfile.cachePath = v;
      if (const char *v = std::getenv("WTC_SOLVER_PROFILE_TOPK")) envProfile.topK = std::atoll(v);
      if (const char *v = std::getenv("WTC_SOLVER_PROFILE_ITERS")) envProfile.iters = std::atoi(v);
      profile = &envProfile;
    }
  }
  if (profile && profile->enable) {
    std::string plog;
    profileCandidates(inputMlir, spec, maxConnectLevel, *profile, sorted, plog);
    if (profile->verbose || std::getenv("WTC_SOLVER_PROFILE_LOG")) std::fputs(plog.c_str(), stderr);
  }
  if (!bestSummaryJson.empty() && !writeBestSummaryJson(spec, arch, sorted, bestSummaryJson, error)) { span.fail(); return 4; }
  if (!candidatesTsv.empty() && !writeCandidatesTsv(sorted, candidatesTsv, error)) { span.fail(); return 4; }
  const Candidate &b = sorted.front();
  best.tileM = b.tileM; best.tileN = b.tileN; best.tileK = b.tileK;
  best.threadTileM = b.threadTileM; best.threadTileN = b.threadTileN;
  error.clear();
  return 0;
}

} // namespace wtc::scheduler
