// libwelder-solver-capi.so: the search entry point the front-end dlopens.  Contract in
// include/welder_solver_capi.h.  Holds no global state, so it tolerates being loaded into
// a private linker namespace and unloaded after every call.
#include "../../../include/welder_solver_capi.h"

#include "wtc_host.h"

#include <algorithm>
#include <cstring>

namespace {
void setError(char *buf, size_t n, const std::string &msg) {
  if (!buf || n == 0) return;
  const size_t k = std::min(n - 1, msg.size());
  std::memcpy(buf, msg.data(), k);
  buf[k] = '\0';
}
} // namespace

extern "C" int welder_solver_solve_typical_chain(const char *input_mlir_path, const char *best_summary_json_path,
                                                 const char *candidates_tsv_path, int64_t max_connect_level, int /*verbose*/,
                                                 int64_t *out_tile_m, int64_t *out_tile_n, int64_t *out_tile_k,
                                                 int64_t *out_thread_tile_m, int64_t *out_thread_tile_n, char *error_buffer,
                                                 size_t error_buffer_size) {
  setError(error_buffer, error_buffer_size, "");
  if (!input_mlir_path || !*input_mlir_path) { setError(error_buffer, error_buffer_size, "input_mlir_path is empty"); return 1; }
  if (!out_tile_m || !out_tile_n || !out_tile_k || !out_thread_tile_m || !out_thread_tile_n) {
    setError(error_buffer, error_buffer_size, "output tile pointers must not be null");
    return 1;
  }
  wtc::scheduler::SearchResult best;
  std::string error;
  const int rc = wtc::scheduler::solveTypicalChain(input_mlir_path, best_summary_json_path ? best_summary_json_path : "",
                                                   candidates_tsv_path ? candidates_tsv_path : "", max_connect_level, best, error);
  if (rc != 0) { setError(error_buffer, error_buffer_size, error); return rc; }
  *out_tile_m = best.tileM; *out_tile_n = best.tileN; *out_tile_k = best.tileK;
  *out_thread_tile_m = best.threadTileM; *out_thread_tile_n = best.threadTileN;
  return 0;
}
