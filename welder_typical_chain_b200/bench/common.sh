# Shared by the harness scripts: locations, the build step, small helpers.
# Environment knobs common to every script (same names as the reference harness, bench/run_ab.sh:7-33):
#   INPUT_MLIR  OUT_BASE  BACKEND_ROOT (alias LEGACY_ROOT)  BACKEND_MODE  MAX_CONNECT_LEVEL
BENCH_DIR="$(cd -- "$(dirname -- "${BASH_SOURCE[0]}")" && pwd)"
PKG_DIR="$(cd -- "${BENCH_DIR}/.." && pwd)"
BACKEND_ROOT="${BACKEND_ROOT:-${PKG_DIR}/backend/welder}"
[[ -n "${LEGACY_ROOT:-}" ]] && BACKEND_ROOT="${LEGACY_ROOT}"
BACKEND_MODE="${BACKEND_MODE:-process_chain}"
MAX_CONNECT_LEVEL="${MAX_CONNECT_LEVEL:-1}"
WTC="${PKG_DIR}/build/wtc-compiler"
PROFILER="${BACKEND_ROOT}/compiler/build/welder-profiler"

die() { echo "error: $*" >&2; exit 2; }

# Build the native host programs and the launch library if anything is missing.
wtc_build() {
  if [[ ! -x "${WTC}" || ! -x "${PROFILER}" || ! -f "${BACKEND_ROOT}/compiler/build/libwelder-compile-capi.so" ]]; then
    make -C "${PKG_DIR}/host" -j >/dev/null || die "building the host programs failed"
  fi
  if [[ ! -f "${PKG_DIR}/libwtc_launch.so" ]]; then
    make -C "${PKG_DIR}/csrc" -j >/dev/null || die "building the launch library failed"
  fi
  [[ -x "${WTC}" ]] || die "wtc-compiler not found: ${WTC}"
}

# wtc <extra args...>: the front-end with the common arguments filled in
wtc() {
  "${WTC}" --input "${INPUT_MLIR}" --backend-root "${BACKEND_ROOT}" "$@"
}
