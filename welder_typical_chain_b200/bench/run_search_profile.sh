#!/usr/bin/env bash
# Tile search with on-device profiling of the best-ranked candidates: every tile shape the
# kernel library has is compiled to a plan, timed by welder-profiler on the GPU, cached, and
# the measured order replaces the model's.  Counterpart of the reference's
# mlir_pipeline/run_paper_schedule_profile_e2e.sh (same solver flags; passes when the cache
# has been produced).
#   INPUT_MLIR  OUT_BASE  TOPK (2)  PROFILE_WARMUP (10)  PROFILE_ITERS (100)  PROFILE_CACHE
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/cfg2_f16_native_4096x1024x1024.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_search_profile}"
TOPK="${TOPK:-2}"
PROFILE_WARMUP="${PROFILE_WARMUP:-10}"
PROFILE_ITERS="${PROFILE_ITERS:-100}"
PROFILE_CACHE="${PROFILE_CACHE:-${OUT_BASE}/profile_cache.tsv}"
[[ -f "${INPUT_MLIR}" ]] || die "input not found: ${INPUT_MLIR}"
wtc_build
mkdir -p "${OUT_BASE}/search"
SOLVER="${BACKEND_ROOT}/compiler/build/welder-solver"
"${SOLVER}" "${INPUT_MLIR}" --enable-generic-problem --enable-tile-propagation --enable-cut-edges \
  --enable-two-level-schedule --require-perfect-tiling=false --enable-register-level-schedule \
  --max-connect-level "${MAX_CONNECT_LEVEL}" \
  --dump-best-summary-json "${OUT_BASE}/search/best_summary.json" \
  --dump-candidates-tsv "${OUT_BASE}/search/candidates.tsv" \
  --enable-profiling --schedule-topk "${TOPK}" --profile-warmup "${PROFILE_WARMUP}" --profile-iters "${PROFILE_ITERS}" \
  --profile-cache "${PROFILE_CACHE}" --profile-profiler-bin "${PROFILER}" --profile-verbose \
  2> "${OUT_BASE}/search/solver.log" | tee "${OUT_BASE}/search/best.txt"
cat "${OUT_BASE}/search/solver.log"
if [[ ! -s "${PROFILE_CACHE}" ]]; then
  echo "FAIL: profiling cache was not produced (or empty): ${PROFILE_CACHE}" >&2
  exit 1
fi
echo "[wtc] measured candidates:"
cut -f1-6,9 "${OUT_BASE}/search/candidates.tsv" | head -n $((TOPK + 1))
echo "PASS: search with on-device profiling verified."
