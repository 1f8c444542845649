// Stage orchestration: canonicalize -> tag -> (search) -> compile -> validate, with the
// reference's tile-source priority (--best-json > search > --tile-* overrides on top >
// built-in defaults) and artifact tree (compiler/pipeline/PipelineRunner.cpp:14-32,57-220).
#include "wtc_host.h"

#include <dlfcn.h>
#if defined(__GLIBC__)
#include <link.h>
#endif

#include <array>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <mutex>
#include <regex>
#include <sstream>

namespace wtc::pipeline {
namespace {

using backend::BackendMode;
using scheduler::SearchResult;

using SolveFn = int (*)(const char *, const char *, const char *, int64_t, int, int64_t *, int64_t *, int64_t *, int64_t *,
                        int64_t *, char *, size_t);
using CompileFn = int (*)(const char *, const char *, const char *, const char *, int64_t, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int, int, char *, size_t);

// ---- search ------------------------------------------------------------------
bool searchByApi(const std::string &input, const backend::ToolchainPaths &tc, const std::filesystem::path &bestSummary,
                 const std::filesystem::path &candidates, const std::filesystem::path &log, int64_t level, bool verbose,
                 SearchResult &result, std::string &diag) {
  if (tc.solverCapiLib.empty()) { diag = "solver C API library not found under: " + tc.buildDir; return false; }
  // A private linker namespace first, so the solver shares no global state with a later
  // in-process compile; the handle is closed after every call.
  void *handle = nullptr;
#if defined(__GLIBC__)
  handle = dlmopen(LM_ID_NEWLM, tc.solverCapiLib.c_str(), RTLD_NOW | RTLD_LOCAL);
#endif
  if (!handle) handle = dlopen(tc.solverCapiLib.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!handle) { diag = std::string("dlopen failed: ") + dlerror(); return false; }
  auto fn = reinterpret_cast<SolveFn>(dlsym(handle, "welder_solver_solve_typical_chain"));
  if (!fn) { diag = "dlsym(welder_solver_solve_typical_chain) failed"; dlclose(handle); return false; }
  std::array<char, 4096> err{};
  int64_t tm = 0, tn = 0, tk = 0, ttm = 0, ttn = 0;
  {
    std::ofstream ofs(log, std::ios::trunc);
    ofs << "[wtc.search.api] lib=" << tc.solverCapiLib << "\n[wtc.search.api] input=" << input << "\n[wtc.search.api] max_connect_level=" << level << "\n";
  }
  const int rc = fn(input.c_str(), bestSummary.c_str(), candidates.c_str(), level, verbose ? 1 : 0, &tm, &tn, &tk, &ttm, &ttn, err.data(), err.size());
  dlclose(handle);
  if (rc != 0) { diag = "backend solver(api) failed, rc=" + std::to_string(rc) + ", error=" + err.data() + ", see " + log.string(); return false; }
  result.tileM = tm; result.tileN = tn; result.tileK = tk; result.threadTileM = ttm; result.threadTileN = ttn;
  return true;
}

bool searchByProcess(const std::string &input, const backend::ToolchainPaths &tc, const std::filesystem::path &bestSummary,
                     const std::filesystem::path &candidates, const std::filesystem::path &log, int64_t level, std::string &diag) {
  if (tc.solverBin.empty()) { diag = "welder-solver not found under: " + tc.buildDir; return false; }
  std::ostringstream cmd;
  cmd << backend::shellQuote(tc.solverBin) << " " << backend::shellQuote(input)
      << " --enable-generic-problem --enable-tile-propagation --enable-cut-edges --enable-two-level-schedule"
      << " --require-perfect-tiling=false --enable-register-level-schedule --max-connect-level " << level
      << " --dump-best-summary-json " << backend::shellQuote(bestSummary.string()) << " --dump-candidates-tsv "
      << backend::shellQuote(candidates.string()) << " > " << backend::shellQuote(log.string()) << " 2>&1";
  const int rc = backend::runShellCommand(cmd.str());
  if (rc != 0) { diag = "backend solver failed, rc=" + std::to_string(rc) + ", see " + log.string(); return false; }
  return true;
}

bool runSearch(const std::string &input, const std::string &backendRoot, const std::filesystem::path &searchDir, BackendMode mode,
               int64_t level, bool verbose, SearchResult &result, std::string &diag) {
  backend::ToolchainPaths tc;
  if (!backend::resolveToolchain(backendRoot, tc, diag)) return false;
  const auto bestSummary = searchDir / "best_summary.json", candidates = searchDir / "candidates.tsv", best = searchDir / "best.json",
             log = searchDir / "solver.log";
  bool ok;
  if (mode == BackendMode::Api) ok = searchByApi(input, tc, bestSummary, candidates, log, level, verbose, result, diag);
  else ok = searchByProcess(input, tc, bestSummary, candidates, log, level, diag);
  if (!ok) return false;
  if (!std::filesystem::exists(bestSummary)) { diag = "solver output missing: " + bestSummary.string(); return false; }
  if (mode != BackendMode::Api && !scheduler::loadBestFromJson(bestSummary.string(), result, diag)) return false;
  return scheduler::writeBestToJson(result, best.string(), diag);
}

// ---- compile -----------------------------------------------------------------
// One cached handle for the process, every call under one mutex, 4 KiB error buffer.
struct CompileApiSession {
  std::mutex mu;
  void *handle = nullptr;
  CompileFn fn = nullptr;
  std::string lib;
  bool compile(const std::string &libPath, const std::string &input, const std::string &outDir, const std::string &compilerBin,
               const SearchResult &t, int64_t level, bool fused, bool verbose, std::string &diag) {
    std::lock_guard<std::mutex> lk(mu);
    if (!handle || lib != libPath) {
      if (handle) dlclose(handle);
      handle = dlopen(libPath.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (!handle) { diag = std::string("dlopen failed: ") + dlerror(); return false; }
      fn = reinterpret_cast<CompileFn>(dlsym(handle, "welder_compile_typical_chain_to_nvvm"));
      if (!fn) { diag = "dlsym(welder_compile_typical_chain_to_nvvm) failed"; dlclose(handle); handle = nullptr; return false; }
      lib = libPath;
    }
    std::array<char, 4096> err{};
    const int rc = fn(input.c_str(), outDir.c_str(), "", compilerBin.c_str(), t.tileM, t.tileN, t.tileK, t.threadTileM, t.threadTileN, level,
                      fused ? 1 : 0, verbose ? 1 : 0, err.data(), err.size());
    if (rc != 0) { diag = "backend compile(api) failed, rc=" + std::to_string(rc) + ", error=" + err.data(); return false; }
    return true;
  }
};
CompileApiSession &compileSession() { static CompileApiSession s; return s; }

bool runCompile(const std::string &input, const std::string &backendRoot, const std::string &outDir, BackendMode mode, const SearchResult &t,
                int64_t level, bool fused, bool verbose, std::string &diag) {
  if (t.tileM <= 0 || t.tileN <= 0 || t.tileK <= 0 || t.threadTileM <= 0 || t.threadTileN <= 0) { diag = "invalid tile sizes (all must be > 0)"; return false; }
  backend::ToolchainPaths tc;
  if (!backend::resolveToolchain(backendRoot, tc, diag)) return false;
  std::filesystem::create_directories(outDir);
  if (mode == BackendMode::Api) {
    if (tc.compileCapiLib.empty()) { diag = "compile C API library not found under: " + tc.buildDir; return false; }
    return compileSession().compile(tc.compileCapiLib, input, outDir, tc.compilerBin, t, level, fused, verbose, diag);
  }
  if (tc.compilerBin.empty()) { diag = "welder-compiler not found under: " + tc.buildDir; return false; }
  const std::string log = (std::filesystem::path(outDir) / "compile.process.log").string();
  std::ostringstream cmd;
  cmd << backend::shellQuote(tc.compilerBin) << " " << backend::shellQuote(input)
      << " --enable-generic-problem --enable-tile-propagation --enable-cut-edges --enable-two-level-schedule --require-perfect-tiling=false"
      << " --force-tile-m " << t.tileM << " --force-tile-n " << t.tileN << " --force-tile-k " << t.tileK
      << " --enable-register-level-schedule --thread-tile-m " << t.threadTileM << " --thread-tile-n " << t.threadTileN
      << " --max-connect-level " << level
      << (fused ? " --reduction-chain-split-broadcast-edges=false --enable-row-reduction-chain-reuse-fusion --enable-row-reduction-input-promotion "
                  "--enable-matmul-softmax-shared-reuse-fusion"
                : " --reduction-chain-split-broadcast-edges=true")
      << " --emit-all-stages --output " << backend::shellQuote((std::filesystem::path(outDir) / "03.after_postbufferize.mlir").string()) << " > "
      << backend::shellQuote(log) << " 2>&1";
  const int rc = backend::runShellCommand(cmd.str());
  if (rc != 0) { diag = "welder-compiler failed, rc=" + std::to_string(rc) + ", see " + log; return false; }
  return true;
}

} // namespace

bool validatePostbufferizeArtifacts(const std::string &artifactDir, std::string &diagnostic) {
  if (artifactDir.empty()) { diagnostic = "artifact dir is empty"; return false; }
  const std::filesystem::path out = artifactDir;
  if (!std::filesystem::exists(out)) { diagnostic = "artifact dir not found: " + artifactDir; return false; }
  const auto postPath = out / "03.after_postbufferize.mlir", launchPath = out / "04.after_workgroup_launch.mlir",
             runnablePath = out / "05.out.nvvm.runnable.mlir";
  if (!std::filesystem::exists(postPath) || !std::filesystem::exists(launchPath) || !std::filesystem::exists(runnablePath)) {
    diagnostic = "expected compiler artifacts are missing under " + artifactDir;
    return false;
  }
  const std::string post = readAll(postPath.string()), launch = readAll(launchPath.string()), runnable = readAll(runnablePath.string());
  if (post.empty() || launch.empty() || runnable.empty()) { diagnostic = "failed to read compiler artifacts under " + artifactDir; return false; }
  // The reference's counters (compiler/runtime/PostbufferizeFixups.cpp:69-85) plus the facts
  // that describe a tcgen05 kernel.
  std::ostringstream r;
  r << "post_matmul_count=" << countContains(post, "linalg.matmul") + countContains(post, "linalg.batch_matmul") << "\n"
    << "launch_kernel_count=" << countContains(launch, "gpu.launch") << "\n"
    << "launch_alloca_count=" << countContains(launch, "memref.alloca") << "\n"
    << "nvvm_mma_sync_count=" << countContains(runnable, "nvvm.mma.sync") << "\n"
    << "ptx_ld_local_count=" << countContains(runnable, "ld.local") << "\n"
    << "ptx_st_local_count=" << countContains(runnable, "st.local") << "\n"
    << "launch_func_count=" << countContains(runnable, "gpu.launch_func") << "\n"
    << "tcgen05_kernel=" << (runnable.find("kernel = \"tc_") != std::string::npos ? 1 : 0) << "\n";
  // kernel facts from the plan attributes: what the counters above meant for the reference's
  // generated code (tensor-core use, on-chip footprint) read off a precompiled tcgen05 kernel
  auto planInt = [&](const char *key) -> long long {
    std::smatch m;
    const std::regex re(std::string("\\b") + key + "\\s*=\\s*(-?[0-9]+)");
    return std::regex_search(runnable, m, re) ? std::stoll(m[1].str()) : 0;
  };
  const bool tc = runnable.find("kernel = \"tc_") != std::string::npos;
  r << "cluster_ctas=" << planInt("cluster_n") << "\n"
    << "threads_per_cta=" << planInt("threads") << "\n"
    << "pipeline_stages=" << planInt("stages") << "\n"
    << "tmem_columns=" << planInt("tmem_columns") << "\n"
    << "workspace_bytes=" << planInt("workspace_bytes") << "\n"
    << "shared_memory_bytes=" << planInt("smem_bytes") << "\n"
    << "registers_per_thread=" << planInt("registers") << "\n"
    << "spill_store_bytes=" << planInt("spill_bytes") << "\n"
    << "stack_frame_bytes=" << planInt("stack_bytes") << "\n"
    << "tcgen05_mma_per_tile=" << (tc ? (planInt("K") + 63) / 64 * 4 : 0) << "\n";
  if (!writeAll((out / "postbufferize_report.txt").string(), r.str())) { diagnostic = "failed to write postbufferize report"; return false; }
  diagnostic.clear();
  return true;
}

int runTypicalChainPipeline(const RunOptions &options) {
  std::string diag;
  if (options.outputDir.empty()) { std::cerr << "error: output dir is empty\n"; return 1; }
  const std::string backendRoot = options.backendRoot.empty() ? backend::defaultBackendRoot() : options.backendRoot;
  const std::filesystem::path root = options.outputDir, irDir = root / "ir", searchDir = root / "search";
  const std::string canonical = (irDir / "01.canonicalized.mlir").string(), tagged = (irDir / "02.tagged.mlir").string(),
                    tagsJson = (irDir / "02.tags.json").string(), bestJson = (searchDir / "best.json").string(),
                    compileDir = (root / (options.fused ? "fused" : "baseline")).string();
  std::filesystem::create_directories(irDir);

  if (options.verbose) std::cout << "[wtc] phase: canonicalize\n";
  if (!ir::canonicalizeMatmulSoftmaxChain(options.inputPath, canonical, diag)) { std::cerr << "error: canonicalize failed: " << diag << "\n"; return 1; }
  if (options.verbose) std::cout << "[wtc] phase: tagging\n";
  if (!ir::tagTypicalChainOps(canonical, tagged, tagsJson, diag)) { std::cerr << "error: tagging failed: " << diag << "\n"; return 1; }
  std::filesystem::create_directories(searchDir);

  SearchResult best;
  bool haveBest = false;
  if (!options.bestJsonPath.empty()) {
    if (options.verbose) std::cout << "[wtc] load best json: " << options.bestJsonPath << "\n";
    if (!scheduler::loadBestFromJson(options.bestJsonPath, best, diag)) { std::cerr << "error: failed to load --best-json: " << diag << "\n"; return 1; }
    haveBest = true;
  }
  if (!haveBest && options.enableSearch) {
    BackendMode searchMode = options.backendMode;
    // full mode keeps search and compile isolated unless --pure-api-full asks for one process
    if (options.backendMode == BackendMode::Api && !options.pureApiFull && options.mode != RunMode::SearchOnly) {
      searchMode = BackendMode::ProcessChain;
      if (options.verbose) std::cout << "[wtc] note: search falls back to process_chain mode for stability before api compile\n";
    } else if (options.backendMode == BackendMode::Api && options.pureApiFull && options.verbose && options.mode != RunMode::SearchOnly) {
      std::cout << "[wtc] note: pure-api-full enabled, run search(api) + compile(api) in one process\n";
    }
    if (options.verbose) std::cout << "[wtc] phase: search (" << backend::toString(options.backendMode) << ")\n";
    if (!runSearch(tagged, backendRoot, searchDir, searchMode, options.maxConnectLevel, options.verbose, best, diag)) {
      std::cerr << "error: search failed: " << diag << "\n";
      return 1;
    }
    haveBest = true;
    if (options.verbose) std::cout << "[wtc] search best: " << bestJson << "\n[wtc] search candidates: " << (searchDir / "candidates.tsv").string() << "\n";
  }
  if (options.tileM > 0 || options.tileN > 0 || options.tileK > 0 || options.threadTileM > 0 || options.threadTileN > 0) {
    if (options.verbose) std::cout << "[wtc] apply tile overrides\n";
    if (options.tileM > 0) best.tileM = options.tileM;
    if (options.tileN > 0) best.tileN = options.tileN;
    if (options.tileK > 0) best.tileK = options.tileK;
    if (options.threadTileM > 0) best.threadTileM = options.threadTileM;
    if (options.threadTileN > 0) best.threadTileN = options.threadTileN;
    haveBest = true;
  }
  if (!haveBest && options.mode == RunMode::SearchOnly) { std::cerr << "error: search-only mode has no result. Provide --best-json or enable search.\n"; return 1; }
  if (!haveBest && !options.enableSearch && options.verbose) std::cout << "[wtc] search disabled, using built-in default tiles\n";
  if (!scheduler::writeBestToJson(best, bestJson, diag)) { std::cerr << "error: failed to persist best.json: " << diag << "\n"; return 1; }
  if (options.verbose)
    std::cout << "[wtc] selected tile=(" << best.tileM << "x" << best.tileN << "x" << best.tileK << ") thread_tile=(" << best.threadTileM << "x"
              << best.threadTileN << ")\n";
  if (options.mode == RunMode::SearchOnly) { std::cout << "[wtc] search completed. best: " << bestJson << "\n"; return 0; }

  if (options.verbose) std::cout << "[wtc] phase: build transform + compile (" << backend::toString(options.backendMode) << ")\n";
  if (!runCompile(tagged, backendRoot, compileDir, options.backendMode, best, options.maxConnectLevel, options.fused, options.verbose, diag)) {
    std::cerr << "error: build/compile failed: " << diag << "\n";
    return 1;
  }
  if (options.verbose) std::cout << "[wtc] phase: validate postbufferize artifacts\n";
  if (!validatePostbufferizeArtifacts(compileDir, diag)) { std::cerr << "error: postbufferize artifact validation failed: " << diag << "\n"; return 1; }
  std::cout << "[wtc] pipeline completed. artifact: " << (std::filesystem::path(compileDir) / "05.out.nvvm.runnable.mlir").string() << "\n";
  return 0;
}

} // namespace wtc::pipeline
