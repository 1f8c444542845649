// "Compile" stage of the B200 build: turn the recognised chain plus a tile choice into
// the artifact set the reference's compile stage leaves behind
// (backend/welder/compiler/driver/WelderCompileSession.cpp:239-329):
//   03.after_postbufferize.mlir     the chain on buffers (what one call reads and writes)
//   04.after_workgroup_launch.mlir  the launch plan: one gpu.launch per kernel, with grid /
//                                   cluster / block / shared- and tensor-memory footprint
//   04c.after_linalg_to_loops.mlir  the per-CTA loop structure of the fused kernel
//   05.out.nvvm.runnable.mlir       the runnable plan the runner (welder-profiler) consumes
// There is no code generation: the kernels are precompiled for sm_100a in the launch
// library, and the plan (kernel family, legalised tiles, workspace) is what
// wtc_plan_query of that library reports for the chain descriptor.
#include "wtc_host.h"

#include "../../../include/wtc_launch.h"

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <sstream>

namespace wtc::transform {
namespace {

const char *kKernelNames[] = {"simt_fused", "tc_cluster", "tc_tiled", "simt_unfused", "tc_unfused"};

std::string moduleDir() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void *>(&moduleDir), &info) && info.dli_fname)
    return std::filesystem::absolute(std::filesystem::path(info.dli_fname)).parent_path().string();
  return ".";
}

int dtypeCode(const std::string &t) { return t == "f16" ? WTC_F16 : WTC_F32; }

std::string memrefType(const ir::ChainSpec &s, int64_t rows, int64_t cols, const std::string &elem, bool batched) {
  std::ostringstream o;
  o << "memref<";
  if (batched) o << s.batch << "x";
  o << rows << "x" << cols << "x" << elem << ">";
  return o.str();
}

struct PlanResult {
  wtc_chain_desc desc;
  wtc_plan_info plan;
};

bool queryPlan(const ir::ChainSpec &spec, const CompileRequest &req, PlanResult &out, std::string &error) {
  const std::string lib = findLaunchLibrary();
  if (lib.empty()) { error = "launch library libwtc_launch.so not found (set WTC_LAUNCH_LIB)"; return false; }
  void *h = dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) { error = std::string("dlopen failed: ") + dlerror(); return false; }
  auto query = reinterpret_cast<int (*)(const wtc_chain_desc *, wtc_plan_info *)>(dlsym(h, "wtc_plan_query"));
  auto lastError = reinterpret_cast<const char *(*)()>(dlsym(h, "wtc_last_error"));
  if (!query || !lastError) { error = "launch library lacks wtc_plan_query"; dlclose(h); return false; }
  wtc_chain_desc &d = out.desc;
  d = wtc_chain_desc();
  d.struct_size = sizeof(wtc_chain_desc);
  d.batch = static_cast<int32_t>(spec.batch);
  d.M = spec.M; d.N = spec.N; d.K = spec.K;
  d.b_batch_stride = spec.bBatched || spec.batch == 1 ? 0 : -1;
  d.in_dtype = dtypeCode(spec.argType);
  if (spec.argType != spec.inType) d.flags |= WTC_FLAG_MATMUL_F16;   // f32 buffers, rounded to f16 before the contraction
  d.out_dtype = dtypeCode(spec.outType);
  d.acc_dtype = dtypeCode(spec.accType);
  d.scale = static_cast<float>(spec.scale);
  d.tile_m = static_cast<int32_t>(req.tileM); d.tile_n = static_cast<int32_t>(req.tileN); d.tile_k = static_cast<int32_t>(req.tileK);
  d.variant = req.fused ? WTC_VARIANT_FUSED : WTC_VARIANT_BASELINE;
  const int rc = query(&d, &out.plan);
  if (rc != 0) error = std::string("wtc_plan_query failed: ") + lastError();
  dlclose(h);
  return rc == 0;
}

std::string postbufferizeText(const ir::ChainSpec &s, const CompileRequest &req) {
  const std::string aT = memrefType(s, s.M, s.K, s.argType, s.batched), bT = memrefType(s, s.K, s.N, s.argType, s.bBatched),
                    oT = memrefType(s, s.M, s.N, s.outType, s.batched);
  const char *mm = s.batched ? "linalg.batch_matmul" : "linalg.matmul";
  std::ostringstream o;
  o << "// wtc stage 03: the chain on buffers (" << (req.fused ? "fused" : "baseline") << " variant)\n"
    << "// requested tile " << req.tileM << "x" << req.tileN << "x" << req.tileK << ", thread tile " << req.threadTileM << "x"
    << req.threadTileN << ", max connect level " << req.maxConnectLevel << "\n"
    << "module {\n  func.func @" << s.funcName << "(%A: " << aT << ", %B: " << bT << ", %Out: " << oT << ") {\n"
    << "    // logits: accumulate " << s.inType << " x " << s.inType << " products in f32"
    << (s.accType == "f16" ? ", round once to f16 (chain spells an f16 matmul result)" : "") << "\n"
    << "    %S = " << mm << " ins(%A, %B : " << aT << ", " << bT << ") -> logits<" << (s.batched ? std::to_string(s.batch) + "x" : "") << s.M << "x"
    << s.N << "xf32>\n";
  if (s.scale != 1.0) o << "    %V = wtc.scale %S {factor = " << s.scale << " : f32}\n";
  if (req.fused)
    o << "    // logits stay on chip: tensor memory -> registers -> shared memory -> %Out\n"
      << "    wtc.row_softmax %" << (s.scale != 1.0 ? "V" : "S") << " -> %Out : " << oT << "  {max, exp, sum, div fused; reductions over d" << (s.batched ? 2 : 1) << "}\n";
  else
    o << "    // baseline: every broadcast edge is cut, intermediates live in global memory\n"
      << "    %C32 = memref.alloc() : memref<" << s.batch * s.M << "x" << s.N << "xf32>\n"
      << "    %max = memref.alloc() : memref<" << s.batch * s.M << "xf32>\n"
      << "    %E = memref.alloc() : memref<" << s.batch * s.M << "x" << s.N << "xf32>\n"
      << "    %sum = memref.alloc() : memref<" << s.batch * s.M << "xf32>\n"
      << "    wtc.row_max %C32 -> %max\n    wtc.exp_sub %C32, %max -> %E\n    wtc.row_sum %E -> %sum\n    wtc.div %E, %sum -> %Out\n";
  o << "    return\n  }\n}\n";
  return o.str();
}

std::string launchText(const ir::ChainSpec &s, const PlanResult &pr) {
  const wtc_plan_info &p = pr.plan;
  std::ostringstream o;
  o << "// wtc stage 04: launch plan for sm_100a (kernel family " << kKernelNames[p.kernel] << ")\n";
  const int64_t rb = (s.M + 127) / 128, nb = (s.N + 255) / 256;
  auto launch = [&](const std::string &name, const std::string &grid, const std::string &cluster, int threads, const std::string &smem,
                    const std::string &note) {
    o << "gpu.launch @" << name << " blocks(" << grid << ") cluster(" << cluster << ") threads(" << threads << ", 1, 1) workgroup(" << smem
      << ")  // " << note << "\n";
  };
  switch (p.kernel) {
    case WTC_KERNEL_TC_CLUSTER:
      launch("fused_tc_kernel_cluster", "min(" + std::to_string(s.batch * rb) + " row blocks, resident clusters) x " + std::to_string(p.cluster_n),
             std::to_string(p.cluster_n) + ", 1, 1", p.threads,
             std::to_string(p.stages) + " stages x 48 KiB operands + 64 KiB f16 staging + 18 KiB row statistics",
             "persistent; tcgen05.mma 128x256x16, " + std::to_string(p.tmem_columns) + " TMEM columns; row (max,sum) swapped through DSMEM");
      break;
    case WTC_KERNEL_TC_TILED:
      launch("fused_tc_kernel_tiled", "min(" + std::to_string(s.batch * rb * nb) + " tiles, SMs)", "1, 1, 1", p.threads,
             std::to_string(p.stages) + " stages x 48 KiB operands + 32 KiB f16 staging",
             "persistent; writes exp(v - tile max) and per-tile (max,sum), workspace " + std::to_string(p.workspace_bytes) + " B");
      launch("rescale_rows_kernel", std::to_string(s.batch * s.M) + " rows", "1, 1, 1", 256, std::to_string(nb * 4) + " B",
             "log-sum-exp over the tiles of a row, rescale in place");
      break;
    case WTC_KERNEL_SIMT_FUSED:
      launch("simt_fused_kernel", "ceil(rows / R)", "1, 1, 1", 256, "R x (64 + N) f32", "exact f32 accumulate, k ascending; one warp per row in the softmax");
      break;
    default:
      launch("unfused_matmul_kernel", "ceil(rows / 8)", "1, 1, 1", 256, "8 x 64 f32", "C32 = scale * A.B -> global");
      launch("rowmax_kernel", "ceil(rows / 8)", "1, 1, 1", 256, "0", "max[M] <- C32");
      launch("exp_kernel", "elementwise", "1, 1, 1", 256, "0", "E <- exp(C32 - max)");
      launch("rowsum_kernel", "ceil(rows / 8)", "1, 1, 1", 256, "0", "sum[M] <- E");
      launch("div_kernel", "elementwise", "1, 1, 1", 256, "0", "Out <- E / sum");
      break;
  }
  return o.str();
}

std::string loopsText(const ir::ChainSpec &s, const PlanResult &pr) {
  const wtc_plan_info &p = pr.plan;
  std::ostringstream o;
  o << "// wtc stage 04c: loop structure per CTA (kernel family " << kKernelNames[p.kernel] << ")\n";
  if (p.kernel == WTC_KERNEL_TC_CLUSTER || p.kernel == WTC_KERNEL_TC_TILED) {
    o << "scf.for %tile = %cta to %tiles step %ctas {            // persistent tile loop, two TMEM accumulators in flight\n"
      << "  scf.for %kb = 0 to " << (s.K + 63) / 64 << " {                          // warp 0: TMA   warp 1: tcgen05.mma\n"
      << "    tma.load  A[128 x 64], B[64 x 256] -> stage[%kb mod " << p.stages << "]   // 128-byte swizzle, mbarrier complete_tx\n"
      << "    tcgen05.mma x4 (M128 N256 K16)  D[tmem] += A[smem] * B[smem]\n"
      << "  }\n"
      << "  // warps 2..9, one row x 128 columns per thread\n"
      << "  tcgen05.ld 128 accumulators -> registers ; release the accumulator\n"
      << "  m = max_j v ; e_j = ex2(v_j - m) ; l = sum_j e_j\n"
      << (p.kernel == WTC_KERNEL_TC_CLUSTER ? "  st.async (m, l) -> every CTA of the cluster ; combine ; p_j = e_j * 2^(m - m_row) / l_row\n"
                                            : "  store (m_tile, l_tile) ; p_j = e_j (normalised later by rescale_rows_kernel)\n")
      << "  f16 -> swizzled shared -> tma.store\n"
      << "}\n";
  } else {
    o << "scf.for %i = %row0 to %row1 {\n  scf.for %j = 0 to " << s.N << " {\n    scf.for %k = 0 to " << s.K
      << " { %acc = fma(A[%i,%k], B[%k,%j], %acc) }\n  }\n  row max ; exp ; row sum ; divide\n}\n";
  }
  return o.str();
}

std::string runnableText(const ir::ChainSpec &s, const CompileRequest &req, const PlanResult &pr) {
  const wtc_plan_info &p = pr.plan;
  char scale[64];
  snprintf(scale, sizeof scale, "%.9g", s.scale);
  std::ostringstream o;
  o << "// wtc stage 05: runnable plan.  The kernels are precompiled for sm_100a in libwtc_launch.so;\n"
    << "// the runner rebuilds the chain descriptor from the attributes below and calls wtc_matmul_softmax_launch.\n"
    << "module attributes {gpu.container_module, wtc.target = \"sm_100a\"} {\n"
    << "  wtc.chain {batch = " << s.batch << ", M = " << s.M << ", N = " << s.N << ", K = " << s.K << ", b_batched = " << (s.bBatched ? 1 : 0)
    << ", arg_dtype = \"" << s.argType << "\", in_dtype = \"" << s.inType << "\", acc_dtype = \"" << s.accType << "\", out_dtype = \"" << s.outType << "\", scale = " << scale << "}\n"
    << "  wtc.tiles {requested_m = " << req.tileM << ", requested_n = " << req.tileN << ", requested_k = " << req.tileK << ", tile_m = " << p.tile_m
    << ", tile_n = " << p.tile_n << ", tile_k = " << p.tile_k << ", thread_tile_m = " << req.threadTileM << ", thread_tile_n = " << req.threadTileN
    << ", substituted = " << p.tile_substituted << "}\n"
    << "  wtc.plan {variant = \"" << (req.fused ? "fused" : "baseline") << "\", kernel = \"" << kKernelNames[p.kernel] << "\", launches = " << p.launches
    << ", cluster_n = " << p.cluster_n << ", threads = " << p.threads << ", stages = " << p.stages << ", tmem_columns = " << p.tmem_columns
    << ", workspace_bytes = " << p.workspace_bytes << ", smem_bytes = " << p.smem_bytes << ", registers = " << p.registers
    << ", spill_bytes = " << p.spill_bytes << ", stack_bytes = " << p.stack_bytes << "}\n"
    << "  func.func @" << s.funcName << "(%A: !wtc.device_ptr, %B: !wtc.device_ptr, %Out: !wtc.device_ptr, %workspace: !wtc.device_ptr) {\n";
  for (int i = 0; i < p.launches; ++i)
    o << "    gpu.launch_func @wtc_kernels::@" << kKernelNames[p.kernel] << "_" << i << " args(%A, %B, %Out, %workspace)\n";
  o << "    return\n  }\n}\n";
  return o.str();
}

// ---- the row-only chains (row softmax of a given matrix; row variance broadcast along the row):
// one fused kernel each, no tiles to choose, no workspace
bool isRowChain(const ir::ChainSpec &s) { return s.kind == "row_softmax" || s.kind == "layernorm_variance"; }

std::string rowChainStage(const ir::ChainSpec &s, int stage) {
  const bool sm = s.kind == "row_softmax";
  const char *kernel = sm ? "row_softmax" : "row_variance";
  const bool warpRows = s.N <= 2048;
  const long long grid = warpRows ? (s.M + 7) / 8 : s.M;
  const std::string t = "memref<" + std::to_string(s.M) + "x" + std::to_string(s.N) + "x" + s.inType + ">";
  char f1[64], f2[64];
  snprintf(f1, sizeof f1, "%.9g", s.meanFactor);
  snprintf(f2, sizeof f2, "%.9g", s.varFactor);
  std::ostringstream o;
  if (stage == 3) {
    o << "// wtc stage 03: the row chain on buffers\nmodule {\n  func.func @" << s.funcName << "(%X: " << t << ", %Out: " << t << ") {\n";
    if (sm) o << "    wtc.row_softmax %X -> %Out : " << t << "  {max, exp, sum, div fused; reduction over d1}\n";
    else o << "    wtc.row_variance %X -> %Out : " << t << "  {sum, mean = " << f1 << " * sum, squared differences, sum, var = " << f2
           << " * sum, broadcast; reductions over d1}\n";
    o << "    return\n  }\n}\n";
  } else if (stage == 4) {
    o << "// wtc stage 04: launch plan for sm_100a (kernel " << kernel << ")\nmodule attributes {gpu.container_module} {\n"
      << "  func.func @" << s.funcName << "(%X: !wtc.device_ptr, %Out: !wtc.device_ptr) {\n"
      << "    gpu.launch blocks(" << grid << ", 1, 1) threads(256, 1, 1) {   // "
      << (warpRows ? "one warp per row, the row in registers between the passes" : "one CTA per row, three passes (the later ones from L2)")
      << "\n      wtc." << kernel << " %X, %Out\n      gpu.terminator\n    }\n    return\n  }\n}\n";
  } else if (stage == 40) {
    o << "// wtc stage 04c: loop structure per " << (warpRows ? "warp" : "CTA") << " (kernel " << kernel << ")\n"
      << "scf.for %row = mine {\n";
    if (sm) o << "  %m = max_j X[%row, j]\n  %e[j] = exp(X[%row, j] - %m)\n  %s = sum_j %e[j]\n  Out[%row, j] = %e[j] / %s\n";
    else o << "  %mean = " << f1 << " * sum_j X[%row, j]\n  %var = " << f2 << " * sum_j (X[%row, j] - %mean)^2\n  Out[%row, j] = %var\n";
    o << "}\n";
  } else {
    o << "// wtc stage 05: runnable plan.  The kernels are precompiled for sm_100a in libwtc_launch.so;\n"
      << "// the runner rebuilds the descriptor from the attributes below and calls wtc_row_chain_launch.\n"
      << "module attributes {gpu.container_module, wtc.target = \"sm_100a\"} {\n"
      << "  wtc.chain {kind = \"" << s.kind << "\", batch = 1, M = " << s.M << ", N = " << s.N << ", K = 0, b_batched = 0, arg_dtype = \"" << s.inType
      << "\", in_dtype = \"" << s.inType << "\", acc_dtype = \"f32\", out_dtype = \"" << s.outType << "\", scale = 1, mean_factor = " << f1
      << ", var_factor = " << f2 << "}\n"
      << "  wtc.plan {variant = \"fused\", kernel = \"" << kernel << "\", launches = 1, cluster_n = 1, threads = 256, stages = 0, tmem_columns = 0, workspace_bytes = 0"
      << ", smem_bytes = " << (warpRows ? 0 : 32) << ", registers = 0, spill_bytes = 0, stack_bytes = 0}\n"
      << "  func.func @" << s.funcName << "(%X: !wtc.device_ptr, %Out: !wtc.device_ptr) {\n"
      << "    gpu.launch_func @wtc_kernels::@" << kernel << "_0 args(%X, %Out)\n    return\n  }\n}\n";
  }
  return o.str();
}

} // namespace

std::string findLaunchLibrary() {
  if (const char *e = std::getenv("WTC_LAUNCH_LIB"); e && *e && std::filesystem::exists(e)) return e;
  std::filesystem::path dir = moduleDir();
  for (int up = 0; up < 6; ++up) {
    const auto cand = dir / "libwtc_launch.so";
    if (std::filesystem::exists(cand)) return cand.string();
    if (!dir.has_parent_path() || dir.parent_path() == dir) break;
    dir = dir.parent_path();
  }
  return "";
}

int emitPostbufferizeStage(const CompileRequest &req, const std::string &outputPath, std::string &error) {
  ir::ChainSpec spec;
  if (!ir::parseChainFile(req.inputMlirPath, spec, error)) return 2;
  if (!writeAll(outputPath, isRowChain(spec) ? rowChainStage(spec, 3) : postbufferizeText(spec, req))) { error = "cannot open output file: " + outputPath; return 2; }
  return 0;
}

int compileChainToPlan(const CompileRequest &req, std::string &error) {
  trace::Span span("compile");
  auto failWith = [&](const std::string &m) { error = m; span.fail(); return 2; };
  if (req.inputMlirPath.empty()) return failWith("input_mlir_path is empty");
  if (req.outDir.empty()) return failWith("out_dir is empty");
  if (req.tileM <= 0 || req.tileN <= 0 || req.tileK <= 0 || req.threadTileM <= 0 || req.threadTileN <= 0) return failWith("invalid tile sizes");
  std::error_code ec;
  std::filesystem::create_directories(req.outDir, ec);
  if (ec) return failWith("failed to create out_dir: " + req.outDir + ", ec=" + std::to_string(ec.value()));
  const std::filesystem::path out = req.outDir;
  ir::ChainSpec spec;
  std::string perr;
  if (!ir::parseChainFile(req.inputMlirPath, spec, perr)) return failWith("chain recogniser: " + perr);
  if (isRowChain(spec)) {
    if (spec.inType != spec.outType) return failWith("row chain: the result must have the argument's element type");
    std::ostringstream rlog;
    rlog << "[wtc.compile] input=" << req.inputMlirPath << "\n[wtc.compile] row chain kind=" << spec.kind << " rows=" << spec.M << " N=" << spec.N
         << " dtype=" << spec.inType << ": one fused kernel, no tile choice, no workspace (requested tile " << req.tileM << "x" << req.tileN << "x"
         << req.tileK << " recorded only)\n";
    if (!writeAll((out / "03.after_postbufferize.mlir").string(), rowChainStage(spec, 3)) ||
        !writeAll((out / "04.after_workgroup_launch.mlir").string(), rowChainStage(spec, 4)) ||
        !writeAll((out / "04c.after_linalg_to_loops.mlir").string(), rowChainStage(spec, 40)) ||
        !writeAll((out / "05.out.nvvm.runnable.mlir").string(), rowChainStage(spec, 5)) ||
        !writeAll((out / "compile.log").string(), rlog.str()))
      return failWith("failed to write compile artifacts under " + req.outDir);
    error.clear();
    return 0;
  }
  PlanResult pr;
  if (!queryPlan(spec, req, pr, perr)) return failWith(perr);

  std::ostringstream log;
  log << "[wtc.compile] input=" << req.inputMlirPath << "\n[wtc.compile] variant=" << (req.fused ? "fused" : "baseline")
      << " kernel=" << kKernelNames[pr.plan.kernel] << " launches=" << pr.plan.launches << "\n[wtc.compile] requested tile " << req.tileM << "x"
      << req.tileN << "x" << req.tileK << " -> used " << pr.plan.tile_m << "x" << pr.plan.tile_n << "x" << pr.plan.tile_k
      << (pr.plan.tile_substituted ? " (requested tile is not legal for this kernel family on sm_100a; substituted)" : "") << "\n"
      << "[wtc.compile] thread tile " << req.threadTileM << "x" << req.threadTileN << " recorded (no meaning for tcgen05 kernels)\n"
      << "[wtc.compile] workspace_bytes=" << pr.plan.workspace_bytes << " cluster_n=" << pr.plan.cluster_n << " stages=" << pr.plan.stages << "\n";
  if (!writeAll((out / "03.after_postbufferize.mlir").string(), postbufferizeText(spec, req)) ||
      !writeAll((out / "04.after_workgroup_launch.mlir").string(), launchText(spec, pr)) ||
      !writeAll((out / "04c.after_linalg_to_loops.mlir").string(), loopsText(spec, pr)) ||
      !writeAll((out / "05.out.nvvm.runnable.mlir").string(), runnableText(spec, req, pr)) ||
      !writeAll((out / "compile.log").string(), log.str()))
    return failWith("failed to write compile artifacts under " + req.outDir);
  error.clear();
  return 0;
}

} // namespace wtc::transform
