#!/usr/bin/env bash
# A/B: compile baseline + fused, time both on the GPU (CUDA events, WARMUP/ITERS launches),
# optionally verify the dumps, and report the speedup.
#   <OUT_BASE>/ab_summary.{tsv,csv}   case avg_ms kernels pattern seed iters warmup out_dir
#   <OUT_BASE>/speedup.tsv            baseline_ms / fused_ms
# Knobs: WARMUP ITERS PATTERN SEED VERIFY VERIFY_RTOL VERIFY_ATOL M (rows to run, default: the chain's).
set -euo pipefail
source "$(dirname -- "${BASH_SOURCE[0]}")/common.sh"
INPUT_MLIR="${INPUT_MLIR:-${PKG_DIR}/mlir/matmul_softmax_chain_f16_native.mlir}"
OUT_BASE="${OUT_BASE:-/tmp/wtc_ab}"
WARMUP="${WARMUP:-10}"; ITERS="${ITERS:-200}"
PATTERN="${PATTERN:-linear}"; SEED="${SEED:-1}"
VERIFY="${VERIFY:-0}"; VERIFY_RTOL="${VERIFY_RTOL:-1e-3}"; VERIFY_ATOL="${VERIFY_ATOL:-1e-3}"
[[ -f "${INPUT_MLIR}" ]] || die "input mlir not found: ${INPUT_MLIR}"
wtc_build
INPUT_MLIR="${INPUT_MLIR}" OUT_BASE="${OUT_BASE}" BACKEND_ROOT="${BACKEND_ROOT}" BACKEND_MODE="${BACKEND_MODE}" \
  MAX_CONNECT_LEVEL="${MAX_CONNECT_LEVEL}" bash "${BENCH_DIR}/run_compile_pair.sh"
[[ -x "${PROFILER}" ]] || die "profiler not found: ${PROFILER}"

summary_tsv="${OUT_BASE}/ab_summary.tsv"; summary_csv="${OUT_BASE}/ab_summary.csv"
printf 'case\tavg_ms\tkernels\tpattern\tseed\titers\twarmup\tout_dir\n' >"${summary_tsv}"
echo "case,avg_ms,kernels,pattern,seed,iters,warmup,out_dir" >"${summary_csv}"
rows_arg=(); [[ -n "${M:-}" ]] && rows_arg=(--m "${M}")

run_case() {
  local name="$1" dir="${OUT_BASE}/$1" plan="${OUT_BASE}/$1/05.out.nvvm.runnable.mlir"
  [[ -f "${plan}" ]] || die "missing compiled artifact for ${name}: ${plan}"
  echo "[run:${name}] perf"
  "${PROFILER}" --warmup="${WARMUP}" --iters="${ITERS}" --init="${PATTERN}" --seed="${SEED}" "${rows_arg[@]}" "${plan}" \
    | tee "${dir}/profile.log" | tail -n 1
  if [[ "${VERIFY}" == "1" ]]; then
    echo "[run:${name}] verify"
    if ! "${PROFILER}" --warmup=0 --iters=1 --init="${PATTERN}" --seed="${SEED}" "${rows_arg[@]}" \
         --dump-last-2d "${dir}/out.bin" "${plan}" >"${dir}/verify_profile.log" 2>&1; then
      echo "[warn:${name}] profiler verify run failed" | tee "${dir}/verify.log"
    elif ! python3 "${BENCH_DIR}/verify.py" --out "${dir}/out.bin" --plan "${plan}" --pattern "${PATTERN}" --seed "${SEED}" \
           --rtol "${VERIFY_RTOL}" --atol "${VERIFY_ATOL}" | tee "${dir}/verify.log"; then
      echo "[warn:${name}] numerical verification failed (see ${dir}/verify.log)"
    fi
  fi
  local avg_ms kernels
  avg_ms="$(grep -o -m 1 'avg_ms=[0-9.eE+-]*' "${dir}/profile.log" | sed 's/avg_ms=//')"
  [[ -n "${avg_ms}" ]] || die "failed to parse avg_ms from ${dir}/profile.log"
  kernels="$(grep -c 'gpu.launch' "${dir}/04.after_workgroup_launch.mlir")"
  printf '%s\t%s\t%s\t%s\t%s\t%s\t%s\t%s\n' "${name}" "${avg_ms}" "${kernels}" "${PATTERN}" "${SEED}" "${ITERS}" "${WARMUP}" "${dir}" >>"${summary_tsv}"
  echo "${name},${avg_ms},${kernels},${PATTERN},${SEED},${ITERS},${WARMUP},${dir}" >>"${summary_csv}"
  echo "summary:${name}: avg_ms=${avg_ms} kernels=${kernels} out_dir=${dir}"
}
run_case baseline
run_case fused
speedup="$(awk -F'\t' '$1=="baseline"{b=$2} $1=="fused"{f=$2} END{if(f+0==0) print "nan"; else printf "%.4f", b/f}' "${summary_tsv}")"
printf 'speedup\t%s\n' "${speedup}" | tee "${OUT_BASE}/speedup.tsv"
echo "done: baseline=${OUT_BASE}/baseline fused=${OUT_BASE}/fused speedup=${speedup}x"
