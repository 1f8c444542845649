/*
 * welder_compile_capi.h -- compile entry points of libwelder-compile-capi.so.
 *
 * welder_compile_typical_chain_to_nvvm: same symbol, argument list and return codes as
 * the reference's backend/welder/compiler/driver/WelderCompileCAPI.h:19-25
 * (implementation driver/WelderCompileCAPI.cpp:20-71): 0 ok, 1 bad arguments, 2 failure;
 * the error buffer is caller-owned and always NUL-terminated; strings are borrowed.
 * It leaves 03.after_postbufferize.mlir, 04.after_workgroup_launch.mlir,
 * 04c.after_linalg_to_loops.mlir, 05.out.nvvm.runnable.mlir and compile.log in out_dir
 * (names of WelderCompileCAPI.h:12-16).  The plugin and compiler-binary paths are accepted
 * and unused: there is no MLIR pass plugin in this build.
 *
 * welderCompilerMain: same name and C++ linkage as driver/WelderCompilerMain.h:4; argv as
 * driver/WelderCompileSession.cpp:167-205 assembles it; safe to call repeatedly in one
 * process (driver/WelderCompiler.cpp:190-193 needs option resets for that; here nothing is
 * global).  Returns 0 on success.
 */
#ifndef WELDER_COMPILE_CAPI_H
#define WELDER_COMPILE_CAPI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
int welderCompilerMain(int argc, char **argv);
extern "C" {
#endif

int welder_compile_typical_chain_to_nvvm(const char *input_mlir_path, const char *out_dir,
                                         const char *workgroup_pass_plugin_path, const char *welder_compiler_bin_path,
                                         int64_t tile_m, int64_t tile_n, int64_t tile_k, int64_t thread_tile_m,
                                         int64_t thread_tile_n, int64_t max_connect_level, int fused, int verbose,
                                         char *error_buffer, size_t error_buffer_size);

#ifdef __cplusplus
}
#endif
#endif /* WELDER_COMPILE_CAPI_H */
