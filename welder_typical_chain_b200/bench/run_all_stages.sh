#!/usr/bin/env bash
# Acceptance run: regression -> compile pair (api) -> pure-api stress -> A/B -> optional perf
# guard; one row per stage in <OUT_BASE>/all_stages_summary.tsv.  RUN_AB=0 skips the GPU stages.
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
OUT_BASE="${OUT_BASE:-/tmp/wtc_all_stages}"
RUN_AB="${RUN_AB:-1}"; RUN_PERF_GUARD="${RUN_PERF_GUARD:-0}"; STRESS_REPEAT="${STRESS_REPEAT:-20}"
mkdir -p "${OUT_BASE}"
SUMMARY="${OUT_BASE}/all_stages_summary.tsv"
printf 'stage\tstatus\tseconds\tlog\n' >"${SUMMARY}"
stage() {
  local name="$1"; shift
  local log="${OUT_BASE}/${name}.log" t0 t1 status=PASS
  t0="$(date +%s)"
  if ! "$@" >"${log}" 2>&1; then status=FAIL; fi
  t1="$(date +%s)"
  printf '%s\t%s\t%s\t%s\n' "${name}" "${status}" "$((t1 - t0))" "${log}" >>"${SUMMARY}"
  echo "[stage:${name}] ${status}"
  [[ "${status}" == PASS ]] || { tail -n 20 "${log}" >&2; exit 1; }
}
stage regression env OUT_BASE="${OUT_BASE}/regression" bash "${BENCH_DIR}/run_regression.sh"
stage compile_pair_api env OUT_BASE="${OUT_BASE}/pair" BACKEND_MODE=api bash "${BENCH_DIR}/run_compile_pair.sh"
stage pure_api_stress env OUT_BASE="${OUT_BASE}/stress" REPEAT="${STRESS_REPEAT}" bash "${BENCH_DIR}/run_pure_api_stress.sh"
if [[ "${RUN_AB}" == "1" ]]; then
  stage ab env OUT_BASE="${OUT_BASE}/ab" VERIFY="${VERIFY:-1}" bash "${BENCH_DIR}/run_ab.sh"
  if [[ "${RUN_PERF_GUARD}" == "1" ]]; then
    stage perf_guard env CURRENT_OUT_BASE="${OUT_BASE}/ab" bash "${BENCH_DIR}/check_perf_guard.sh"
  fi
fi
echo "[wtc] all stages passed"
echo "  summary: ${SUMMARY}"
