// Tool discovery, the three backend modes and the tracer.
//   api           dlopen the C-API libraries and call them in-process
//                 (compiler/scheduler/SearchBackendApi.cpp:46-89, compiler/transform/CompileApiSession.cpp:13-73)
//   process_chain spawn welder-solver / welder-compiler (SearchBackendProcessChain.cpp, BuildCutEdgesTransformProcessChain.cpp)
//   shell         kept as an alias of process_chain: there are no wrapper scripts to run in this build
#include "wtc_host.h"

#include <dlfcn.h>
#if defined(__GLIBC__)
#include <link.h>
#endif
#include <unistd.h>

#include <array>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <mutex>
#include <sstream>

namespace wtc {

namespace trace {
namespace {
double nowMs() {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
std::mutex g_traceMu;
} // namespace
Span::Span(const char *name) : name_(name), t0_(nowMs()) {}
Span::~Span() {
  const char *path = std::getenv("WTC_TRACE_FILE");
  if (!path || !*path) return;
  std::lock_guard<std::mutex> lk(g_traceMu);
  std::ofstream ofs(path, std::ios::app);
  if (!ofs) return;
  ofs << "{\"name\": \"" << name_ << "\", \"dur_ms\": " << (nowMs() - t0_) << ", \"ok\": " << (ok_ ? "true" : "false")
      << ", \"pid\": " << getpid() << "}\n";
}
} // namespace trace

namespace backend {

bool parseBackendMode(const std::string &text, BackendMode &mode, std::string &diagnostic) {
  diagnostic.clear();
  if (text == "shell") { mode = BackendMode::Shell; return true; }
  if (text == "api") { mode = BackendMode::Api; return true; }
  if (text == "process_chain" || text == "subprocess_pipeline" || text == "inprocess") { mode = BackendMode::ProcessChain; return true; }
  diagnostic = "unknown backend mode: " + text + " (expected shell|process_chain|api)";
  return false;
}

const char *toString(BackendMode mode) {
  switch (mode) {
    case BackendMode::Shell: return "shell";
    case BackendMode::Api: return "api";
    default: return "process_chain";
  }
}

std::string shellQuote(const std::string &s) {
  std::string out = "'";
  for (char c : s) {
    if (c == '\'') out += "'\\''";
    else out.push_back(c);
  }
  out.push_back('\'');
  return out;
}

int runShellCommand(const std::string &cmd) {
  const int rc = std::system(cmd.c_str());
  if (rc == -1) return -1;
  if (WIFEXITED(rc)) return WEXITSTATUS(rc);
  return rc;
}

std::string defaultBackendRoot() {
  if (const char *e = std::getenv("WTC_BACKEND_ROOT"); e && *e) return e;
  std::error_code ec;
  const auto exe = std::filesystem::read_symlink("/proc/self/exe", ec);
  if (!ec) {
    const auto cand = exe.parent_path().parent_path() / "backend" / "welder";
    if (std::filesystem::exists(cand)) return cand.string();
  }
  return "backend/welder";
}

bool resolveToolchain(const std::string &backendRoot, ToolchainPaths &p, std::string &diagnostic) {
  if (backendRoot.empty()) { diagnostic = "backend root is empty"; return false; }
  const std::filesystem::path root = backendRoot;
  if (!std::filesystem::exists(root)) { diagnostic = "backend root not found: " + backendRoot; return false; }
  const std::filesystem::path build = root / "compiler" / "build";
  p.backendRoot = root.string();
  p.buildDir = build.string();
  auto pick = [&](const char *name) { const auto f = build / name; return std::filesystem::exists(f) ? f.string() : std::string(); };
  p.solverBin = pick("welder-solver");
  p.compilerBin = pick("welder-compiler");
  p.profilerBin = pick("welder-profiler");
  p.solverCapiLib = pick("libwelder-solver-capi.so");
  p.compileCapiLib = pick("libwelder-compile-capi.so");
  diagnostic.clear();
  return true;
}

} // namespace backend
} // namespace wtc
