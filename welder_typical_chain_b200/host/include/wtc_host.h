// Host side of the B200 build of the typical chain (Matmul -> row Softmax): chain
// recogniser, tile chooser, plan emitter, backend sessions and the pipeline driver.
// Plain C++17; the only native dependency is libdl.  Mirrors the reference
// front-end's stage structure (canonicalize -> tag -> search -> compile ->
// validate, compiler/pipeline/PipelineRunner.cpp:57-220) with every MLIR/LLVM
// dependency replaced by a small recogniser for the one chain this build serves.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace wtc {

// ------------------------------------------------------------------ chain IR
namespace ir {

// What the recogniser extracts from `func @main`.
struct ChainSpec {
  // which chain the function spells: "matmul_softmax" (the operator this build serves), or one of
  // the row-only chains of the reference's backend inputs: "row_softmax"
  // (backend/welder/mlir_pipeline/softmax_row_chain.mlir) and "layernorm_variance"
  // (backend/welder/mlir_pipeline/layernorm_variance_chain.mlir); for those K = 0
  std::string kind = "matmul_softmax";
  double meanFactor = 0.0, varFactor = 0.0;   // layernorm_variance: the constants applied to the two row sums
  std::string funcName = "main";
  int64_t batch = 1, M = 0, N = 0, K = 0;
  bool batched = false;        // linalg.batch_matmul + softmax over the last of 3 dims
  bool bBatched = false;       // B carries the batch dimension too
  std::string inType = "f32";  // element type of the matmul's operands
  std::string argType = "f32"; // element type of the function arguments: inType, or f32 when the chain rounds
                               // its arguments to f16 first (mlir_pipeline/matmul_softmax_chain_f16_matmul.mlir:18-44)
  std::string accType = "f32"; // element type of the matmul's outs
  std::string outType = "f32"; // element type of the function result
  double scale = 1.0;          // product of constant arith.mulf factors between matmul and softmax
  bool namedSoftmax = false;   // input used linalg.softmax (else the max/exp/sum/div generics)
  int matmulCount = 0, genericCount = 0, reductionCount = 0, expCount = 0, divCount = 0;
};

// Parses the restricted grammar (see chain_ir.cpp).  Comments are ignored, so the
// tagged file parses like the canonical one.
bool parseChain(const std::string &mlirText, ChainSpec &spec, std::string &diag);
// The dataflow matcher behind parseChain (chain_match.cpp): `text` has comments stripped and
// aliases expanded.
bool matchChain(const std::string &text, ChainSpec &spec, std::string &diag);
bool parseChainFile(const std::string &path, ChainSpec &spec, std::string &diag);
std::string chainToJson(const ChainSpec &spec);

// Stage 1: writes <out> with linalg.softmax decomposed into max/exp/sum/div
// generics (text rewrite), plus 01.canonicalize.log and chain.json beside it.
// Accepts iff the result has a matmul, math.exp and arith.divf and no
// linalg.softmax (same checks as compiler/ir/ChainCanonicalize.cpp:145-159).
bool canonicalizeMatmulSoftmaxChain(const std::string &inputPath, const std::string &outputPath,
                                    std::string &diagnostic);
// Stage 2: comment tags + 02.tags.json (compiler/ir/Tagging.cpp:50-159).
bool tagTypicalChainOps(const std::string &inputPath, const std::string &outputPath,
                        const std::string &tagsJsonPath, std::string &diagnostic);

} // namespace ir

// ------------------------------------------------------------------ tiles / search
namespace scheduler {

// Defaults of compiler/include/wtc/scheduler/Search.h:11-17.
struct SearchResult {
  int64_t tileM = 32, tileN = 64, tileK = 16, threadTileM = 2, threadTileN = 2;
};

bool loadBestFromJson(const std::string &jsonPath, SearchResult &result, std::string &diagnostic);
bool writeBestToJson(const SearchResult &result, const std::string &jsonPath, std::string &diagnostic);

// One candidate of the B200 tile chooser.
struct Candidate {
  int64_t tileM, tileN, tileK, threadTileM, threadTileN;
  int stages, clusterN;
  bool implemented;            // the kernel library has this tile shape
  double score;                // L2->SM operand bytes x waves (lower is better)
  double estimatedLatencyUs;
  double profiledMs = -1.0;    // measured on the device by the profiling pass; -1: not measured
  double bytesA, bytesB, bytesC, bytesCut;
};

struct ArchModel {             // sm_100a, per CTA / per chip
  int64_t smemBytes = 232448, numSM = 148, warpSize = 32, tmemColumns = 512;
  double tensorTflops = 2250.0, l2TBps = 14.0, hbmTBps = 6.5;
};

// Enumerates legal sm_100a tiles for the chain, scores them, sorts (implemented
// first, then score) and returns the list; never empty for a valid chain.
std::vector<Candidate> enumerateCandidates(const ir::ChainSpec &spec, const ArchModel &arch,
                                           int64_t maxConnectLevel);
bool writeBestSummaryJson(const ir::ChainSpec &spec, const ArchModel &arch, const std::vector<Candidate> &sorted,
                          const std::string &path, std::string &error);
bool writeCandidatesTsv(const std::vector<Candidate> &sorted, const std::string &path, std::string &error);
// On-device profiling of the best-ranked candidates (the reference's `d.Profile` step:
// solver/WelderSolver.cpp:202-213,479-513; compile + run welder-profiler per candidate,
// solver/WelderSolverProfileCompileAndRun.h:137-2453; append-only `key<TAB>ms` cache,
// solver/WelderSolverProfileRetryHelpers.h:796-833).
struct ProfileOptions {
  bool enable = false;
  int64_t topK = 8;            // --schedule-topk: how many implemented candidates are measured
  int warmup = 10, iters = 100;
  std::string profilerBin;     // empty: welder-profiler beside this module
  std::string cachePath;       // empty: no disk cache
  bool verbose = false;        // keeps the temporary plans
};
// Fills `profiledMs` of up to topK implemented candidates (cache first, then compile the
// plan and run the profiler binary), then moves the measured ones to the front ordered by
// time.  Returns how many carry a measurement; candidates whose run fails stay unmeasured.
int profileCandidates(const std::string &inputMlir, const ir::ChainSpec &spec, int64_t maxConnectLevel,
                      const ProfileOptions &opts, std::vector<Candidate> &sorted, std::string &log);
std::string buildProfileKey(const ir::ChainSpec &spec, const Candidate &c, int64_t maxConnectLevel);
// parse + enumerate (+ profile) + write; the shared body of the solver C API and CLI.
int solveTypicalChain(const std::string &inputMlir, const std::string &bestSummaryJson,
                      const std::string &candidatesTsv, int64_t maxConnectLevel, SearchResult &best,
                      std::string &error, const ProfileOptions *profile = nullptr);

} // namespace scheduler

// ------------------------------------------------------------------ compile (plan emission)
namespace transform {

struct CompileRequest {
  std::string inputMlirPath, outDir;
  int64_t tileM = 0, tileN = 0, tileK = 0, threadTileM = 0, threadTileN = 0, maxConnectLevel = 1;
  bool fused = true, verbose = false;
};
// Writes 03/04/04c/05 + compile.log under outDir.  The kernel plan comes from
// wtc_plan_query of the launch library.  rc 0 ok, 2 failure (error filled).
int compileChainToPlan(const CompileRequest &req, std::string &error);
// Only the first stage (the 03 file), as `welder-compiler ... --output <path>` does.
int emitPostbufferizeStage(const CompileRequest &req, const std::string &outputPath, std::string &error);
std::string findLaunchLibrary();   // WTC_LAUNCH_LIB, else next to / above the calling module

} // namespace transform

// ------------------------------------------------------------------ backends + pipeline
namespace backend {

enum class BackendMode { Shell, ProcessChain, Api };
bool parseBackendMode(const std::string &text, BackendMode &mode, std::string &diagnostic);
const char *toString(BackendMode mode);
std::string shellQuote(const std::string &s);
int runShellCommand(const std::string &cmd);

struct ToolchainPaths {
  std::string backendRoot, buildDir;
  std::string solverBin, compilerBin, profilerBin, solverCapiLib, compileCapiLib;
};
// <root>/compiler/build/{welder-solver,welder-compiler,welder-profiler,libwelder-*-capi.so}
bool resolveToolchain(const std::string &backendRoot, ToolchainPaths &paths, std::string &diagnostic);
std::string defaultBackendRoot();   // WTC_BACKEND_ROOT, else <dir of this executable>/../backend/welder

} // namespace backend

namespace pipeline {

enum class RunMode { Full, SearchOnly, CompileOnly };

struct RunOptions {
  std::string inputPath;
  std::string outputDir = "/tmp/wtc_out";
  std::string backendRoot;                 // empty: backend::defaultBackendRoot()
  std::string bestJsonPath;
  int64_t maxConnectLevel = 1;
  int64_t tileM = 0, tileN = 0, tileK = 0, threadTileM = 0, threadTileN = 0;
  bool enableSearch = true;
  bool fused = true;
  backend::BackendMode backendMode = backend::BackendMode::ProcessChain;
  bool pureApiFull = false;
  RunMode mode = RunMode::Full;
  bool verbose = false;
};

int runTypicalChainPipeline(const RunOptions &options);
bool validatePostbufferizeArtifacts(const std::string &artifactDir, std::string &diagnostic);

} // namespace pipeline

// ------------------------------------------------------------------ tracing
// JSON-lines spans for the host stages (one object per line: name, dur_ms, ok),
// written to $WTC_TRACE_FILE when set.  Same idea as the reference's Tracer
// (backend/welder/compiler/common/WelderTrace.h:29-216), host stages only.
namespace trace {
class Span {
public:
  explicit Span(const char *name);
  ~Span();
  void fail() { ok_ = false; }
private:
  const char *name_;
  double t0_;
  bool ok_ = true;
};
} // namespace trace

// shared small helpers
std::string readAll(const std::string &path);
bool writeAll(const std::string &path, const std::string &content);
int countContains(const std::string &text, const std::string &needle);

} // namespace wtc
