/*
 * welder_solver_capi.h -- search entry point of libwelder-solver-capi.so.
 *
 * Same symbol, argument list and return codes as the reference's
 * backend/welder/compiler/solver/WelderSolverCAPI.h:19-24 (implementation
 * solver/WelderSolverCAPI.cpp:104-196): 0 ok, 1 bad arguments, 2 input could not be
 * opened / recognised, 3 no candidates, 4 I/O failure.  All strings are borrowed; the
 * caller-owned error buffer is always NUL-terminated.  Writes best_summary.json
 * (problem / arch / best{tileM,tileN,tileK,threadTileM,threadTileN,score,...}) and the
 * 13-column candidates.tsv of the reference's C-API flavour (WelderSolverCAPI.cpp:40-100).
 * The front-end loads the library into a private linker namespace when it can and
 * closes it after each call (compiler/scheduler/SearchBackendApi.cpp:46-89), so the
 * library keeps no process-global state.
 */
#ifndef WELDER_SOLVER_CAPI_H
#define WELDER_SOLVER_CAPI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int welder_solver_solve_typical_chain(const char *input_mlir_path, const char *best_summary_json_path,
                                      const char *candidates_tsv_path, int64_t max_connect_level, int verbose,
                                      int64_t *out_tile_m, int64_t *out_tile_n, int64_t *out_tile_k,
                                      int64_t *out_thread_tile_m, int64_t *out_thread_tile_n, char *error_buffer,
                                      size_t error_buffer_size);

#ifdef __cplusplus
}
#endif
#endif /* WELDER_SOLVER_CAPI_H */
